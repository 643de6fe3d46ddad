// Rotary position encoding of q and k, fused with the write of k and v into the
// paged cache.
//
// q, k, v of a token lie side by side in one row of the fused projection's
// output: [q heads | k heads | v heads], each head `head_dim` wide.  q is rotated
// in place; k is rotated and v copied into this layer's pages.  Angles are
// position * inv_freq in 32-bit, cos and sin in 32-bit (liteinfer/models/llama.py:
// 78-86 computes them in float32 too, then rounds the tables to the model type;
// here the tables are never rounded, only the rotated result is).  Pairing is
// half-split: dimension j pairs with j + rotary_dim/2 (llama.py:89-102).
// Dimensions from rotary_dim on pass through unrotated.
//
// Values may have another size than keys (`v_dim`): the row is then [q heads | k heads | v heads of v_dim] and the
// value pool's last axis is v_dim.  `cs_scale` multiplies every cosine and sine (1 for a plain rotation).
//
// A page holds `page_size` tokens of every KV head: pool[page][kv_head][slot][dim].
// The page of a token is block_table[seq][position / page_size]; a negative entry
// (a page already given back) skips the write.
//
// li_head_norm_rope_kv_write does the same for an attention whose q and k pass a root-mean-square norm per head
// before the rotation (one weight vector of head_dim for all q heads, one for all k heads), and whose values may
// be blended with another layer's values of the same token before they are stored:
//     q_h <- rot(w_q * q_h / sqrt(mean(q_h^2) + eps));  k likewise;  v <- (1 - lambda) v + lambda v_other
// The row may be wider than q, k and v (further columns of a fused projection follow them).  Statistics, the
// blend and the rotation are 32-bit; each result is rounded once.
//
// `norm_flags`: bit 0, q and k are divided by their root mean square also where no weight is given; bit 1, the norm
// (and its weight) comes behind the rotation instead of in front of it.  `cs_scale` multiplies every cosine and sine.
//
// li_sigmoid_gate_heads multiplies head h of every row of x by sigmoid(gate[row, h]) in place; li_sigmoid_gate
// every element by the sigmoid of its own gate.
#include "common.cuh"

namespace li {

constexpr int kPrepWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
head_norm_rope_kv_write_kernel(T* __restrict__ qkv, size_t row_stride, const int* __restrict__ positions,
                               const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                               int table_stride, T* __restrict__ k_pool, T* __restrict__ v_pool,
                               const float* __restrict__ inv_freq, int heads, int kv_heads, int head_dim,
                               int rotary_dim, int page_size, int num_pages, int v_dim,
                               const T* __restrict__ q_norm, const T* __restrict__ k_norm, float norm_eps,
                               const T* __restrict__ v_other, size_t v_other_stride,
                               const float* __restrict__ lambda, int norm_flags, float cs_scale) {
  extern __shared__ float shared[];  // cos[half], sin[half], then one head per warp
  const bool unit = norm_flags & 1, after = norm_flags & 2;
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  grid_launch_dependents();
  const int pos = positions[t];
  const int half = rotary_dim / 2;
  float* cosv = shared;
  float* sinv = shared + half;
  float* head = shared + rotary_dim + warp * head_dim;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = __fmul_rn((float)pos, inv_freq[i]);
    cosv[i] = cosf(angle) * cs_scale;
    sinv[i] = sinf(angle) * cs_scale;
  }
  const int seq = seq_of_token[t];
  const int page = seq < 0 ? -1 : block_table[(size_t)seq * table_stride + pos / page_size];
  const bool store = page >= 0 && page < num_pages;
  const int slot = pos % page_size;
  const float mix = lambda != nullptr ? lambda[0] : 0.f;
  grid_dependency_wait();           // q, k and v come from the projection before this kernel
  __syncthreads();

  T* row = qkv + (size_t)t * row_stride;
  for (int h = warp; h < heads + kv_heads; h += kPrepWarps) {
    const bool is_q = h < heads;
    const T* w = is_q ? q_norm : k_norm;
    T* p = row + (size_t)h * head_dim;
    float ss = 0.f;
    for (int j = lane; j < head_dim; j += 32) {
      const float x = to_float(p[j]);
      head[j] = x;
      ss = fmaf(x, x, ss);
    }
    const bool normed = w != nullptr || unit;
    if (normed && !after) {
      const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)head_dim + norm_eps);
      for (int j = lane; j < head_dim; j += 32) head[j] = head[j] * inv * (w != nullptr ? to_float(w[j]) : 1.0f);
    }
    __syncwarp();
    T* dst = is_q ? p : k_pool + (((size_t)page * kv_heads + (h - heads)) * page_size + slot) * head_dim;
    if (is_q || store) {
      // With the norm behind the rotation the head is rotated twice: once for its sum of squares, once to be stored.
      float inv = 1.0f;
      for (int pass = (normed && after) ? 0 : 1; pass < 2; ++pass) {
        float ss2 = 0.f;
        for (int j = lane; j < head_dim; j += 32) {
          float r;
          if (j < half) r = rotate_lo(head[j], head[j + half], cosv[j], sinv[j]);
          else if (j < rotary_dim) r = rotate_hi(head[j - half], head[j], cosv[j - half], sinv[j - half]);
          else r = head[j];
          if (pass == 0) ss2 = fmaf(r, r, ss2);
          else dst[j] = from_float<T>((normed && after) ? r * inv * (w != nullptr ? to_float(w[j]) : 1.0f) : r);
        }
        if (pass == 0) inv = 1.0f / sqrtf(warp_sum(ss2) / (float)head_dim + norm_eps);
      }
    }
    __syncwarp();
  }
  if (!store) return;
  const T* vrow = row + (size_t)(heads + kv_heads) * head_dim;
  const T* orow = v_other != nullptr ? v_other + (size_t)t * v_other_stride : nullptr;
  for (int w = threadIdx.x; w < kv_heads * v_dim; w += blockDim.x) {
    const int h = w / v_dim, j = w - h * v_dim;
    float v = to_float(vrow[w]);
    if (orow != nullptr) v = fmaf(mix, to_float(orow[w]), (1.0f - mix) * v);
    v_pool[(((size_t)page * kv_heads + h) * page_size + slot) * v_dim + j] = from_float<T>(v);
  }
}

// The same, a 16-byte vector of neighbouring dimensions a thread: `group` = head_dim / N threads share a head (a power
// of two up to 32, so a head never straddles warps), add up its squares with shuffles, and fetch the rotation's
// partner vector (half a rotary width away: a whole number of vectors) from the lane that holds it.  All items of
// a token are independent loads, so many are in flight at once.
template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
head_norm_rope_kv_write_vec_kernel(T* __restrict__ qkv, size_t row_stride, const int* __restrict__ positions,
                                   const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                   int table_stride, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                   const float* __restrict__ inv_freq, int heads, int kv_heads, int head_dim,
                                   int rotary_dim, int page_size, int num_pages, int v_dim,
                                   const T* __restrict__ q_norm, const T* __restrict__ k_norm, float norm_eps,
                                   const T* __restrict__ v_other, size_t v_other_stride,
                                   const float* __restrict__ lambda, int group_shift, int norm_flags, float cs_scale) {
  constexpr int N = Vec16<T>::N;
  extern __shared__ float shared[];  // cos[half], sin[half]
  const bool unit = norm_flags & 1, after = norm_flags & 2;
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  grid_launch_dependents();
  const int pos = positions[t];
  const int half = rotary_dim / 2;
  float* cosv = shared;
  float* sinv = shared + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = __fmul_rn((float)pos, inv_freq[i]);
    cosv[i] = cosf(angle) * cs_scale;
    sinv[i] = sinf(angle) * cs_scale;
  }
  const int seq = seq_of_token[t];
  const int page = seq < 0 ? -1 : block_table[(size_t)seq * table_stride + pos / page_size];
  const bool store = page >= 0 && page < num_pages;
  const int slot = pos % page_size;
  const float mix = lambda != nullptr ? lambda[0] : 0.f;
  grid_dependency_wait();           // q, k and v come from the projection before this kernel
  __syncthreads();

  T* row = qkv + (size_t)t * row_stride;
  const int group = 1 << group_shift;
  const int qk_items = (heads + kv_heads) << group_shift;
  const int apart = half / N;       // lanes between the two vectors of a rotated pair
  for (int base = 0; base < qk_items; base += kPrepWarps * 32) {
    const int item = base + threadIdx.x;
    const bool active = item < qk_items;         // a head's lanes are active together
    const int h = active ? item >> group_shift : 0, j0 = (item & (group - 1)) * N;
    const bool is_q = h < heads;
    T* p = row + (size_t)h * head_dim + j0;
    float x[N];
#pragma unroll
    for (int e = 0; e < N; ++e) x[e] = 0.f;
    if (active) unpack16(load16(p), x);
    const T* w = is_q ? q_norm : k_norm;
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < N; ++e) ss = fmaf(x[e], x[e], ss);
    for (int o = group >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // by every lane of the warp
    const bool normed = w != nullptr || unit;
    float wv[N];
#pragma unroll
    for (int e = 0; e < N; ++e) wv[e] = 1.0f;
    if (w != nullptr) unpack16(load16(w + j0), wv);
    if (normed && !after) {
      const float inv = 1.0f / sqrtf(ss / (float)head_dim + norm_eps);
#pragma unroll
      for (int e = 0; e < N; ++e) x[e] = x[e] * inv * wv[e];
    }
    // Both halves of a pair are x * cos + partner * (-+ sin), and a dimension that is not rotated is x * 1 +
    // x * 0: the lane fetches its eight cosines and sines (the sign in them) by 16-byte reads once, and every
    // element is the same two products and one sum, rounded as `rotate_lo` / `rotate_hi` round them.
    const int from = j0 < half ? lane + apart : (j0 < rotary_dim ? lane - apart : lane);
    float c[N], sn[N];
    if (j0 < rotary_dim) {
      const int at = j0 < half ? j0 : j0 - half;
      const float sign = j0 < half ? -1.0f : 1.0f;
#pragma unroll
      for (int e = 0; e < N; e += 4) {
        const float4 cv = *reinterpret_cast<const float4*>(cosv + at + e);
        const float4 sv = *reinterpret_cast<const float4*>(sinv + at + e);
        c[e] = cv.x; c[e + 1] = cv.y; c[e + 2] = cv.z; c[e + 3] = cv.w;
        sn[e] = sign * sv.x; sn[e + 1] = sign * sv.y; sn[e + 2] = sign * sv.z; sn[e + 3] = sign * sv.w;
      }
    } else {
#pragma unroll
      for (int e = 0; e < N; ++e) { c[e] = 1.0f; sn[e] = 0.f; }
    }
    Vec16<T> result;
    float r[N];
#pragma unroll
    for (int e = 0; e < N; ++e) {
      const float y = __shfl_sync(0xffffffffu, x[e], from);
      r[e] = j0 < rotary_dim ? __fadd_rn(__fmul_rn(x[e], c[e]), __fmul_rn(y, sn[e])) : x[e];
    }
    if (normed && after) {        // the norm behind the rotation: the root mean square of what was rotated
      float ss2 = 0.f;
#pragma unroll
      for (int e = 0; e < N; ++e) ss2 = fmaf(r[e], r[e], ss2);
      for (int o = group >> 1; o > 0; o >>= 1) ss2 += __shfl_xor_sync(0xffffffffu, ss2, o);
      const float inv = 1.0f / sqrtf(ss2 / (float)head_dim + norm_eps);
#pragma unroll
      for (int e = 0; e < N; ++e) r[e] = r[e] * inv * wv[e];
    }
#pragma unroll
    for (int e = 0; e < N; ++e) result.set(e, r[e]);
    if (active && (is_q || store)) {
      T* dst = is_q ? p : k_pool + (((size_t)page * kv_heads + (h - heads)) * page_size + slot) * head_dim + j0;
      store16(dst, result);
    }
  }
  if (!store) return;
  const T* vrow = row + (size_t)(heads + kv_heads) * head_dim;
  const T* orow = v_other != nullptr ? v_other + (size_t)t * v_other_stride : nullptr;
  for (int w = threadIdx.x * N; w < kv_heads * v_dim; w += kPrepWarps * 32 * N) {
    const int h = w / v_dim, j = w - h * v_dim;
    Vec16<T> v = load16(vrow + w);
    if (orow != nullptr) {
      float a[N], b[N];
      unpack16(v, a);
      unpack16(load16(orow + w), b);
#pragma unroll
      for (int e = 0; e < N; ++e) v.set(e, fmaf(mix, b[e], (1.0f - mix) * a[e]));
    }
    store16(v_pool + (((size_t)page * kv_heads + h) * page_size + slot) * v_dim + j, v);
  }
}

// x [tokens, heads * size] in 16-byte vectors (size a multiple of the vector's length).
template <typename T>
__global__ void sigmoid_gate_heads_vec_kernel(T* __restrict__ x, const T* __restrict__ gate, size_t gate_stride,
                                              size_t tokens, int heads, int size) {
  constexpr int N = Vec16<T>::N;
  grid_dependency_wait();
  const size_t width = (size_t)heads * size / N, total = tokens * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width;
    const int h = (int)((i - t * width) * N / size);
    const float g = 1.0f / (1.0f + expf(-to_float(gate[t * gate_stride + h])));
    Vec16<T> v = load16(x + i * N);
    float a[N];
    unpack16(v, a);
#pragma unroll
    for (int e = 0; e < N; ++e) v.set(e, a[e] * g);
    store16(x + i * N, v);
  }
}

template <typename T>
__global__ void sigmoid_gate_heads_kernel(T* __restrict__ x, const T* __restrict__ gate, size_t gate_stride,
                                          size_t tokens, int heads, int size) {
  grid_dependency_wait();
  const size_t width = (size_t)heads * size, total = tokens * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width;
    const int h = (int)((i - t * width) / size);
    const float g = to_float(gate[t * gate_stride + h]);
    x[i] = from_float<T>(to_float(x[i]) * (1.0f / (1.0f + expf(-g))));
  }
}

// x [tokens, width] *= sigmoid(gate [tokens, width]) element by element; the vector form reads 16 bytes of each.
template <typename T, bool kVec>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, const T* __restrict__ gate, size_t gate_stride, size_t tokens,
                                    int width) {
  constexpr int N = kVec ? Vec16<T>::N : 1;
  grid_dependency_wait();
  const size_t per_row = (size_t)width / N, total = tokens * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / per_row, c = (i - t * per_row) * N;
    if (kVec) {
      Vec16<T> v = load16(x + t * width + c);
      float a[Vec16<T>::N], g[Vec16<T>::N];
      unpack16(v, a);
      unpack16(load16(gate + t * gate_stride + c), g);
#pragma unroll
      for (int e = 0; e < Vec16<T>::N; ++e) v.set(e, a[e] * (1.0f / (1.0f + expf(-g[e]))));
      store16(x + t * width + c, v);
    } else {
      const float g = to_float(gate[t * gate_stride + c]);
      x[t * width + c] = from_float<T>(to_float(x[t * width + c]) * (1.0f / (1.0f + expf(-g))));
    }
  }
}

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                     int table_stride, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                     const float* __restrict__ inv_freq, int heads, int kv_heads, int head_dim,
                                     int rotary_dim, int page_size, int num_pages, int v_dim, float cs_scale) {
  extern __shared__ float cs[];  // cos[half], sin[half]
  const int t = blockIdx.x;
  grid_launch_dependents();
  const int pos = positions[t];   // positions, tables and inv_freq are inputs of the step, not of a kernel
  const int half = rotary_dim / 2;
  float* cosv = cs;
  float* sinv = cs + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = __fmul_rn((float)pos, inv_freq[i]);
    cosv[i] = cs_scale == 1.0f ? cosf(angle) : __fmul_rn(cosf(angle), cs_scale);
    sinv[i] = cs_scale == 1.0f ? sinf(angle) : __fmul_rn(sinf(angle), cs_scale);
  }
  const int seq = seq_of_token[t];
  const int page = seq < 0 ? -1 : block_table[(size_t)seq * table_stride + pos / page_size];   // a row of padding belongs to no sequence
  grid_dependency_wait();           // q, k and v come from the projection before this kernel
  __syncthreads();

  const int row_width = (heads + kv_heads) * head_dim + kv_heads * v_dim;
  T* row = qkv + (size_t)t * row_width;

  // q: rotate in place.  Work item = (head, pair index or pass-through dim).
  const int pass = head_dim - rotary_dim;
  const int per_head = half;  // rotated pairs per head; pass-through dims stay as they are
  for (int w = threadIdx.x; w < heads * per_head; w += blockDim.x) {
    const int h = w / per_head, i = w - h * per_head;
    T* p = row + h * head_dim;
    const float a = to_float(p[i]), b = to_float(p[i + half]);
    p[i] = from_float<T>(rotate_lo(a, b, cosv[i], sinv[i]));
    p[i + half] = from_float<T>(rotate_hi(a, b, cosv[i], sinv[i]));
  }
  (void)pass;

  if (page < 0 || page >= num_pages) return;
  const int slot = pos % page_size;

  const T* krow = row + heads * head_dim;
  const T* vrow = krow + kv_heads * head_dim;
  for (int w = threadIdx.x; w < kv_heads * head_dim; w += blockDim.x) {
    const int h = w / head_dim, j = w - h * head_dim;
    const size_t dst = (((size_t)page * kv_heads + h) * page_size + slot) * head_dim + j;
    float kv;
    if (j < half) {
      kv = rotate_lo(to_float(krow[w]), to_float(krow[w + half]), cosv[j], sinv[j]);
    } else if (j < rotary_dim) {
      kv = rotate_hi(to_float(krow[w - half]), to_float(krow[w]), cosv[j - half], sinv[j - half]);
    } else {
      kv = to_float(krow[w]);
    }
    k_pool[dst] = from_float<T>(kv);
  }
  for (int w = threadIdx.x; w < kv_heads * v_dim; w += blockDim.x) {
    const int h = w / v_dim, j = w - h * v_dim;
    v_pool[(((size_t)page * kv_heads + h) * page_size + slot) * v_dim + j] = vrow[w];
  }
}

// The same with 16-byte accesses, for bfloat16 with every dimension rotated and halves that are multiples of
// eight: one work item is eight pairs (j, j + half) of one head, or eight values of v.
__global__ void rope_kv_write_vec_kernel(bf16* __restrict__ qkv, const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                         int table_stride, bf16* __restrict__ k_pool, bf16* __restrict__ v_pool,
                                         const float* __restrict__ inv_freq, int heads, int kv_heads, int head_dim,
                                         int page_size, int num_pages) {
  extern __shared__ float cs[];  // cos[half], sin[half]
  const int t = blockIdx.x;
  grid_launch_dependents();
  const int pos = positions[t];
  const int half = head_dim / 2;
  float* cosv = cs;
  float* sinv = cs + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = __fmul_rn((float)pos, inv_freq[i]);
    cosv[i] = cosf(angle);
    sinv[i] = sinf(angle);
  }
  const int seq = seq_of_token[t];
  const int page = seq < 0 ? -1 : block_table[(size_t)seq * table_stride + pos / page_size];   // a row of padding belongs to no sequence
  grid_dependency_wait();
  __syncthreads();

  bf16* row = qkv + (size_t)t * (heads + 2 * kv_heads) * head_dim;
  const bool store = page >= 0 && page < num_pages;
  const int slot = pos % page_size;
  const int per_head = half / 8;                       // work items per rotated head
  const int rotated = (heads + kv_heads) * per_head;   // q heads, then k heads
  const int copies = kv_heads * (head_dim / 8);        // v
  for (int w = threadIdx.x; w < rotated + copies; w += blockDim.x) {
    if (w < rotated) {
      const int h = w / per_head, j = (w - h * per_head) * 8;
      bf16* p = row + h * head_dim + j;
      const Vec16<bf16> a = load16(p), b = load16(p + half);
      Vec16<bf16> lo, hi;
      rotate_eight(a, b, cosv + j, sinv + j, lo, hi);
      if (h < heads) {
        store16(p, lo);
        store16(p + half, hi);
      } else if (store) {
        bf16* dst = k_pool + (((size_t)page * kv_heads + (h - heads)) * page_size + slot) * head_dim + j;
        store16(dst, lo);
        store16(dst + half, hi);
      }
    } else if (store) {
      const int c = w - rotated;
      const int h = c / (head_dim / 8), j = (c % (head_dim / 8)) * 8;
      const bf16* src = row + (heads + kv_heads + h) * head_dim + j;
      store16(v_pool + (((size_t)page * kv_heads + h) * page_size + slot) * head_dim + j, load16(src));
    }
  }
}

}  // namespace li

using namespace li;

// inv_freq may be null with rotary_dim 0: nothing is rotated, k and v are only stored.
LI_EXPORT int li_rope_kv_write(int dtype, void* qkv, const int* positions, const int* seq_of_token,
                               const int* block_table, int table_stride, void* k_pool, void* v_pool,
                               const float* inv_freq, int tokens, int heads, int kv_heads, int head_dim,
                               int rotary_dim, int page_size, int num_pages, int v_dim, float cs_scale,
                               cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (v_dim < 1) return LI_ERR_UNSUPPORTED;
  if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return LI_ERR_UNSUPPORTED;
  if (rotary_dim > 0 && inv_freq == nullptr) return LI_ERR_UNSUPPORTED;
  const size_t smem = (size_t)rotary_dim * sizeof(float);
  if (smem > 48 * 1024) return LI_ERR_UNSUPPORTED;
  const int block = 256;
  if (dtype == kBFloat16 && rotary_dim == head_dim && head_dim % 16 == 0 && v_dim == head_dim && cs_scale == 1.0f &&
      aligned16(qkv) && aligned16(k_pool) && aligned16(v_pool))
    return (int)launch_pdl(tokens, rope_kv_write_vec_kernel, dim3(tokens), dim3(block), smem, stream, (bf16*)qkv,
                           positions, seq_of_token, block_table, table_stride, (bf16*)k_pool, (bf16*)v_pool, inv_freq,
                           heads, kv_heads, head_dim, page_size, num_pages);
  if (dtype == kFloat32)
    return (int)launch_pdl(tokens, rope_kv_write_kernel<float>, dim3(tokens), dim3(block), smem, stream, (float*)qkv,
                           positions, seq_of_token, block_table, table_stride, (float*)k_pool, (float*)v_pool,
                           inv_freq, heads, kv_heads, head_dim, rotary_dim, page_size, num_pages, v_dim, cs_scale);
  return (int)launch_pdl(tokens, rope_kv_write_kernel<bf16>, dim3(tokens), dim3(block), smem, stream, (bf16*)qkv, positions,
                         seq_of_token, block_table, table_stride, (bf16*)k_pool, (bf16*)v_pool, inv_freq, heads,
                         kv_heads, head_dim, rotary_dim, page_size, num_pages, v_dim, cs_scale);
}

// q_norm / k_norm: null = that projection is not normalised.  v_other with lambda: the stored values are
// (1 - lambda[0]) v + lambda[0] v_other[t]; null = v as it is.  num_pages 0: nothing is stored (q is still
// normalised and rotated).
LI_EXPORT int li_head_norm_rope_kv_write(int dtype, void* qkv, size_t row_stride, const int* positions,
                                         const int* seq_of_token, const int* block_table, int table_stride,
                                         void* k_pool, void* v_pool, const float* inv_freq, int tokens, int heads,
                                         int kv_heads, int head_dim, int rotary_dim, int page_size, int num_pages,
                                         int v_dim, const void* q_norm, const void* k_norm, float norm_eps,
                                         const void* v_other, size_t v_other_stride, const float* lambda,
                                         int norm_flags, float cs_scale, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (v_dim < 1 || head_dim < 1) return LI_ERR_UNSUPPORTED;
  if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return LI_ERR_UNSUPPORTED;
  if (rotary_dim > 0 && inv_freq == nullptr) return LI_ERR_UNSUPPORTED;
  if ((v_other == nullptr) != (lambda == nullptr)) return LI_ERR_UNSUPPORTED;
  {
    // Vectors of 16 bytes where each lies within one head and one side of the rotation, a head's vectors fit in a
    // warp, and every pointer and stride is a multiple of 16 bytes.
    const int n = dtype == kFloat32 ? 4 : 8;
    const int group = head_dim / n;
    const bool pow2 = head_dim % n == 0 && group >= 1 && group <= 32 && (group & (group - 1)) == 0;
    const bool fits = pow2 && (rotary_dim / 2) % n == 0 && v_dim % n == 0 && row_stride % n == 0 &&
                      (v_other == nullptr || v_other_stride % n == 0) && aligned16(qkv) && aligned16(k_pool) &&
                      aligned16(v_pool) && aligned16(q_norm) && aligned16(k_norm) && aligned16(v_other) &&
                      (size_t)rotary_dim * sizeof(float) <= 48 * 1024;
    if (fits) {
      int shift = 0;
      while ((1 << shift) < group) ++shift;
      const size_t cs = (size_t)rotary_dim * sizeof(float);
      if (dtype == kFloat32)
        return (int)launch_pdl(tokens, head_norm_rope_kv_write_vec_kernel<float>, dim3(tokens), dim3(kPrepWarps * 32), cs,
                               stream, (float*)qkv, row_stride, positions, seq_of_token, block_table, table_stride,
                               (float*)k_pool, (float*)v_pool, inv_freq, heads, kv_heads, head_dim, rotary_dim,
                               page_size, num_pages, v_dim, (const float*)q_norm, (const float*)k_norm, norm_eps,
                               (const float*)v_other, v_other_stride, lambda, shift, norm_flags, cs_scale);
      return (int)launch_pdl(tokens, head_norm_rope_kv_write_vec_kernel<bf16>, dim3(tokens), dim3(kPrepWarps * 32), cs,
                             stream, (bf16*)qkv, row_stride, positions, seq_of_token, block_table, table_stride,
                             (bf16*)k_pool, (bf16*)v_pool, inv_freq, heads, kv_heads, head_dim, rotary_dim, page_size,
                             num_pages, v_dim, (const bf16*)q_norm, (const bf16*)k_norm, norm_eps,
                             (const bf16*)v_other, v_other_stride, lambda, shift, norm_flags, cs_scale);
    }
  }
  const size_t smem = ((size_t)rotary_dim + (size_t)kPrepWarps * head_dim) * sizeof(float);
  if (smem > 48 * 1024) return LI_ERR_UNSUPPORTED;
  if (dtype == kFloat32)
    return (int)launch_pdl(tokens, head_norm_rope_kv_write_kernel<float>, dim3(tokens), dim3(kPrepWarps * 32), smem,
                           stream, (float*)qkv, row_stride, positions, seq_of_token, block_table, table_stride,
                           (float*)k_pool, (float*)v_pool, inv_freq, heads, kv_heads, head_dim, rotary_dim, page_size,
                           num_pages, v_dim, (const float*)q_norm, (const float*)k_norm, norm_eps,
                           (const float*)v_other, v_other_stride, lambda, norm_flags, cs_scale);
  return (int)launch_pdl(tokens, head_norm_rope_kv_write_kernel<bf16>, dim3(tokens), dim3(kPrepWarps * 32), smem, stream,
                         (bf16*)qkv, row_stride, positions, seq_of_token, block_table, table_stride, (bf16*)k_pool,
                         (bf16*)v_pool, inv_freq, heads, kv_heads, head_dim, rotary_dim, page_size, num_pages, v_dim,
                         (const bf16*)q_norm, (const bf16*)k_norm, norm_eps, (const bf16*)v_other, v_other_stride,
                         lambda, norm_flags, cs_scale);
}

LI_EXPORT int li_sigmoid_gate_heads(int dtype, void* x, const void* gate, size_t gate_stride, int tokens, int heads,
                                    int size, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads < 1 || size < 1) return LI_ERR_UNSUPPORTED;
  const int n = dtype == kFloat32 ? 4 : 8;
  if (size % n == 0 && aligned16(x)) {
    const size_t vectors = (size_t)tokens * heads * size / n;
    const dim3 vgrid((unsigned)((vectors + 255) / 256 < 8192 ? (vectors + 255) / 256 : 8192));
    if (dtype == kFloat32)
      return (int)launch_pdl(tokens, sigmoid_gate_heads_vec_kernel<float>, vgrid, dim3(256), 0, stream, (float*)x,
                             (const float*)gate, gate_stride, (size_t)tokens, heads, size);
    return (int)launch_pdl(tokens, sigmoid_gate_heads_vec_kernel<bf16>, vgrid, dim3(256), 0, stream, (bf16*)x,
                           (const bf16*)gate, gate_stride, (size_t)tokens, heads, size);
  }
  const size_t total = (size_t)tokens * heads * size;
  const dim3 grid((unsigned)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192));
  if (dtype == kFloat32)
    return (int)launch_pdl(tokens, sigmoid_gate_heads_kernel<float>, grid, dim3(256), 0, stream, (float*)x,
                           (const float*)gate, gate_stride, (size_t)tokens, heads, size);
  return (int)launch_pdl(tokens, sigmoid_gate_heads_kernel<bf16>, grid, dim3(256), 0, stream, (bf16*)x,
                         (const bf16*)gate, gate_stride, (size_t)tokens, heads, size);
}

// x [tokens, width] (contiguous) *= sigmoid(gate [tokens, width]) (rows gate_stride apart), in place; 32-bit inside.
LI_EXPORT int li_sigmoid_gate(int dtype, void* x, const void* gate, size_t gate_stride, int tokens, int width,
                              cudaStream_t stream) {
  if (tokens <= 0 || width <= 0) return 0;
  const int n = dtype == kFloat32 ? 4 : 8;
  const bool vec = width % n == 0 && gate_stride % n == 0 && aligned16(x) && aligned16(gate);
  const size_t total = (size_t)tokens * width / (vec ? n : 1);
  const dim3 grid((unsigned)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192));
#define LI_GATE(T, V)                                                                                              \
  return (int)launch_pdl(tokens, sigmoid_gate_kernel<T, V>, grid, dim3(256), 0, stream, (T*)x, (const T*)gate,     \
                         gate_stride, (size_t)tokens, width)
  if (dtype == kFloat32) { if (vec) LI_GATE(float, true); LI_GATE(float, false); }
  if (vec) LI_GATE(bf16, true);
  LI_GATE(bf16, false);
#undef LI_GATE
}
