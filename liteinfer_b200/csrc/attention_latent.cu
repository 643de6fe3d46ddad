// Latent attention: every head attends over ONE shared entry per token, [latent (c) | rotated key part (r)].
//
// A token's keys and values are low-rank: key_h = [W_uk,h latent | shared rotated part], value_h = W_uv,h latent.
// The cache therefore keeps only the normalised latent and the rotated part, and the products with W_uk and W_uv
// move to the query's side ("absorbed" form):
//
//     score_h(i, j) = ( (W_uk,h^T q_h,plain)(i) . latent(j) + q_h,rot(i) . shared(j) ) * scale
//     out_h(i)      = W_uv,h ( sum_j p_h(i, j) latent(j) )
//
// so attention is multi-query attention over entries of c + r numbers whose first c are also the values.
// The softmax's denominator may hold one more term per head, exp(sink_h), that belongs to no key ("sink").
// Scores, maxima, sums, the accumulator, angles, cosines and sines are 32-bit.
//
// Kernels here:
//   latent_prep        per token: RMS norm of the query latent (written out for the next product), RMS norm of the
//                      key/value latent and the rotation of the shared key part, both stored into the token's page.
//   latent_attention   SIMT, any sizes and both dtypes: block = (query tile, head chunk, sequence); a warp takes
//                      one (query, head) row at a time and walks its keys 32 at a time from position 0, so the
//                      order of every sum depends on the row's position only, never on how the batch was cut.
//   gate_heads         out[t, h, :] = v[h, t, :] * sigmoid(gate[t, h, :]): the output gate, and the transposition
//                      back to token-major rows.
//
// A page holds `page_size` entries: pool[page][slot][c + r]; the page of a token is block_table[seq][pos / page_size].
#include "common.cuh"

namespace li {

// ------------------------------------------------------------------------------------------ prep
template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T* __restrict__ proj, int proj_stride, int q_off, int q_rank, int kv_off, int kv_rank,
                   int rot_dim, int rot_dims, const float* __restrict__ q_weight, const float* __restrict__ kv_weight,
                   float eps, const float* __restrict__ inv_freq, const int* __restrict__ positions,
                   const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int table_stride,
                   T* __restrict__ pool, int page_size, int num_pages, T* __restrict__ q_out, float cs_scale) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  grid_launch_dependents();
  const int pos = positions[t];
  const int seq = seq_of_token[t];
  int page = -1;
  if (kv_off >= 0 && seq >= 0 && num_pages > 0) page = block_table[(size_t)seq * table_stride + pos / page_size];
  grid_dependency_wait();
  const T* row = proj + (size_t)t * proj_stride;

  // The query latent: x / sqrt(mean(x^2) + eps) * w.
  if (q_out) {
    float ss = 0.f;
    for (int d = threadIdx.x; d < q_rank; d += blockDim.x) {
      const float v = to_float(row[q_off + d]);
      ss = fmaf(v, v, ss);
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    T* o = q_out + (size_t)t * q_rank;
    for (int d = threadIdx.x; d < q_rank; d += blockDim.x)
      o[d] = from_float<T>(__fmul_rn(__fmul_rn(to_float(row[q_off + d]), inv), q_weight[d]));
  }
  if (page < 0 || page >= num_pages) return;      // a layer that reads another layer's entries, or a row of padding

  T* entry = pool + ((size_t)page * page_size + pos % page_size) * (kv_rank + rot_dim);
  float ss = 0.f;
  for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
    const float v = to_float(row[kv_off + d]);
    ss = fmaf(v, v, ss);
  }
  const float inv = rsqrtf(block_sum(ss, scratch) / (float)kv_rank + eps);
  for (int d = threadIdx.x; d < kv_rank; d += blockDim.x)
    entry[d] = from_float<T>(__fmul_rn(__fmul_rn(to_float(row[kv_off + d]), inv), kv_weight[d]));
  // The shared key part: pairs (i, i + rot_dims / 2) of its first rot_dims numbers turn, the rest pass.
  const T* shared = row + kv_off + kv_rank;
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = __fmul_rn((float)pos, inv_freq[i]);
    const float c = cosf(angle) * cs_scale, s = sinf(angle) * cs_scale;
    const float a = to_float(shared[i]), b = to_float(shared[i + half]);
    entry[kv_rank + i] = from_float<T>(rotate_lo(a, b, c, s));
    entry[kv_rank + i + half] = from_float<T>(rotate_hi(a, b, c, s));
  }
  for (int i = rot_dims + threadIdx.x; i < rot_dim; i += blockDim.x) entry[kv_rank + i] = shared[i];
}

// ------------------------------------------------------------------------------------- attention
constexpr int kMaxLatent = 1024;            // most values per entry the SIMT kernel accumulates (16 or 32 per lane)
constexpr int kLatentQueriesPerBlock = 4;
constexpr int kLatentHeadsPerBlock = 8;

template <typename T, int kPerLane>
__global__ void __launch_bounds__(256)
latent_attention_kernel(const T* __restrict__ q_lat, long q_lat_head_stride, int q_lat_token_stride,
                        const T* __restrict__ q_raw, int q_raw_token_stride, int q_raw_head_stride, int q_rot_off,
                        T* __restrict__ out, long out_head_stride, int out_token_stride,
                        const T* __restrict__ pool, const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ query_start_loc, const int* __restrict__ context_lens,
                        const float* __restrict__ inv_freq, const float* __restrict__ sink, int heads, int kv_rank,
                        int rot_dim, int rot_dims, int page_size, int num_pages, float scale, int window,
                        float cs_scale) {
  extern __shared__ float q_smem[];  // [warps][kv_rank + rot_dim]
  const int seq = blockIdx.z;
  grid_launch_dependents();
  const int q_begin = query_start_loc[seq], q_len = query_start_loc[seq + 1] - q_begin;
  const int tile_start = blockIdx.x * kLatentQueriesPerBlock;
  if (tile_start >= q_len) return;
  const int ctx = context_lens[seq];
  const int head0 = blockIdx.y * kLatentHeadsPerBlock;
  const int tile_h = min(kLatentHeadsPerBlock, heads - head0);
  const int tile_q = min(kLatentQueriesPerBlock, q_len - tile_start);
  const int rows = tile_q * tile_h;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int entry_dim = kv_rank + rot_dim;
  float* qs = q_smem + warp * entry_dim;
  const int* table = block_table + (size_t)seq * table_stride;
  const int half = rot_dims / 2;
  grid_dependency_wait();

  for (int row = warp; row < rows; row += nwarps) {
    const int qi = tile_start + row / tile_h;           // query index within the sequence's queries
    const int head = head0 + row % tile_h;
    const int qpos = ctx - q_len + qi;                  // absolute position of this query
    const int token = q_begin + qi;
    const T* ql = q_lat + (size_t)head * q_lat_head_stride + (size_t)token * q_lat_token_stride;
    const T* qr = q_raw + (size_t)token * q_raw_token_stride + (size_t)head * q_raw_head_stride + q_rot_off;
    __syncwarp();
    for (int d = lane; d < kv_rank; d += 32) qs[d] = to_float(ql[d]);
    for (int i = lane; i < half; i += 32) {
      const float angle = __fmul_rn((float)qpos, inv_freq[i]);
      const float c = cosf(angle) * cs_scale, s = sinf(angle) * cs_scale;
      const float a = to_float(qr[i]), b = to_float(qr[i + half]);
      // The rotated query takes the rounding a stored tensor of the engine's dtype would give it, as the key's does.
      qs[kv_rank + i] = round_to<T>(rotate_lo(a, b, c, s));
      qs[kv_rank + i + half] = round_to<T>(rotate_hi(a, b, c, s));
    }
    for (int i = rot_dims + lane; i < rot_dim; i += 32) qs[kv_rank + i] = to_float(qr[i]);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) acc[i] = 0.f;

    // With a window the walk starts at the first visible key rounded down to a multiple of 32: the order of every
    // sum still depends on the row's position only.
    const int first = window > 0 ? max(qpos - window + 1, 0) : 0;
    for (int base = (first / 32) * 32; base <= qpos; base += 32) {
      const int kpos = base + lane;
      long erow = -1;       // index of this lane's entry inside the pool: page * page_size + slot
      float s = -INFINITY;
      if (kpos >= first && kpos <= qpos) {
        const int page = table[kpos / page_size];
        if (page >= 0 && page < num_pages) {
          erow = (long)page * page_size + kpos % page_size;
          const T* kp = pool + (size_t)erow * entry_dim;
          float dot = 0.f;
          for (int d = 0; d < entry_dim; ++d) dot = fmaf(qs[d], to_float(kp[d]), dot);
          s = dot * scale;
        }
      }
      const float m_new = fmaxf(m, warp_max(s));
      if (m_new == -INFINITY) continue;
      const float p = erow >= 0 ? expf(s - m_new) : 0.f;
      const float alpha = expf(m - m_new);  // m = -inf on the first chunk gives 0
      l = l * alpha + warp_sum(p);
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) acc[i] *= alpha;
      const float p_store = round_to<T>(p);   // the probability as an operand of the engine's dtype
      unsigned live = __ballot_sync(0xffffffffu, erow >= 0);
      while (live) {
        const int j = __ffs(live) - 1;
        live &= live - 1;
        const float pj = __shfl_sync(0xffffffffu, p_store, j);
        const long vr = __shfl_sync(0xffffffffu, erow, j);
        const T* vp = pool + (size_t)vr * entry_dim;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
          const int d = lane + 32 * i;
          if (d < kv_rank) acc[i] = fmaf(pj, to_float(vp[d]), acc[i]);
        }
      }
      m = m_new;
    }
    if (sink) {       // one more term of the denominator: it has no key, no value, and is not scaled
      const float sk = sink[head];
      const float m_new = fmaxf(m, sk);
      const float alpha = expf(m - m_new);
      l = l * alpha + expf(sk - m_new);
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) acc[i] *= alpha;
    }
    T* orow = out + (size_t)head * out_head_stride + (size_t)token * out_token_stride;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < kv_rank) orow[d] = from_float<T>(acc[i] * inv);
    }
  }
}

// ------------------------------------------------------------------------------------------ gate
template <typename T>
__global__ void gate_heads_kernel(const T* __restrict__ v, const T* __restrict__ gate, int gate_stride,
                                  T* __restrict__ out, int tokens, int heads, int vdim) {
  grid_dependency_wait();
  grid_launch_dependents();
  const size_t n = (size_t)tokens * heads * vdim;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int e = (int)(i % vdim);
    const int h = (int)((i / vdim) % heads);
    const size_t t = i / ((size_t)vdim * heads);
    float s = 1.0f;
    if (gate) s = 1.0f / (1.0f + expf(-to_float(gate[t * gate_stride + (size_t)h * vdim + e])));
    out[i] = from_float<T>(to_float(v[((size_t)h * tokens + t) * vdim + e]) * s);
  }
}

}  // namespace li

using namespace li;

// proj [tokens, proj_stride]: the query's down projection at columns [q_off, q_off + q_rank), the key/value down
// projection ([latent | shared key part]) at [kv_off, kv_off + kv_rank + rot_dim); kv_off < 0: the layer makes
// no entries of its own.  q_out [tokens, q_rank] (null: skipped).  pool [num_pages, page_size, kv_rank + rot_dim];
// num_pages 0: nothing is stored.  inv_freq [rot_dims / 2] float; q_weight, kv_weight float.  cos_sin_scale multiplies
// every cosine and sine of the rotation.
LI_EXPORT int li_latent_prep(int dtype, const void* proj, int proj_stride, int q_off, int q_rank, int kv_off,
                             int kv_rank, int rot_dim, int rot_dims, const float* q_weight, const float* kv_weight,
                             float eps, const float* inv_freq, const int* positions, const int* seq_of_token,
                             const int* block_table, int table_stride, void* pool, int page_size, int num_pages,
                             void* q_out, int tokens, float cos_sin_scale, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1)) return LI_ERR_UNSUPPORTED;
  cudaError_t e;
  if (dtype == kFloat32)
    e = launch_pdl(tokens, latent_prep_kernel<float>, dim3(tokens), dim3(128), 0, stream, (const float*)proj,
                   proj_stride, q_off, q_rank, kv_off, kv_rank, rot_dim, rot_dims, q_weight, kv_weight, eps, inv_freq,
                   positions, seq_of_token, block_table, table_stride, (float*)pool, page_size, num_pages,
                   (float*)q_out, cos_sin_scale);
  else
    e = launch_pdl(tokens, latent_prep_kernel<bf16>, dim3(tokens), dim3(128), 0, stream, (const bf16*)proj,
                   proj_stride, q_off, q_rank, kv_off, kv_rank, rot_dim, rot_dims, q_weight, kv_weight, eps, inv_freq,
                   positions, seq_of_token, block_table, table_stride, (bf16*)pool, page_size, num_pages,
                   (bf16*)q_out, cos_sin_scale);
  return (int)e;
}

// q_lat: the absorbed queries, head h of token t at q_lat + h * q_lat_head_stride + t * q_lat_token_stride
// (kv_rank numbers).  q_raw: the query projection, the part of head h of token t that turns at
// q_raw + t * q_raw_token_stride + h * q_raw_head_stride + q_rot_off (rot_dim numbers, not yet rotated).
// out: like q_lat.  sink [heads] float or null.  window > 0: a query at position p reads the keys at
// p - window + 1 ... p.  cos_sin_scale multiplies every cosine and sine of the query's rotation.
LI_EXPORT int li_latent_attention(int dtype, const void* q_lat, long q_lat_head_stride, int q_lat_token_stride,
                                  const void* q_raw, int q_raw_token_stride, int q_raw_head_stride, int q_rot_off,
                                  void* out, long out_head_stride, int out_token_stride, const void* pool,
                                  const int* block_table, int table_stride, const int* query_start_loc,
                                  const int* context_lens, const float* inv_freq, const float* sink, int num_seqs,
                                  int max_q_len, int heads, int kv_rank, int rot_dim, int rot_dims, int page_size,
                                  int num_pages, float scale, int window, float cos_sin_scale,
                                  cudaStream_t stream) {
  if (num_seqs == 0 || max_q_len == 0) return 0;
  if (kv_rank < 1 || kv_rank > kMaxLatent || rot_dim < 0 || rot_dims > rot_dim || (rot_dims & 1)) return LI_ERR_UNSUPPORTED;
  if (num_seqs > 65535) return LI_ERR_UNSUPPORTED;
  const int threads = 256;
  const dim3 grid((max_q_len + kLatentQueriesPerBlock - 1) / kLatentQueriesPerBlock,
                  (heads + kLatentHeadsPerBlock - 1) / kLatentHeadsPerBlock, num_seqs);
  const size_t smem = (size_t)(threads / 32) * (kv_rank + rot_dim) * sizeof(float);
  cudaError_t e;
#define LI_LATENT_LAUNCH(T, N)                                                                                        \
  e = launch_pdl(max_q_len, latent_attention_kernel<T, N>, grid, dim3(threads), smem, stream, (const T*)q_lat,        \
                 q_lat_head_stride, q_lat_token_stride, (const T*)q_raw, q_raw_token_stride, q_raw_head_stride,       \
                 q_rot_off, (T*)out, out_head_stride, out_token_stride, (const T*)pool, block_table, table_stride,    \
                 query_start_loc, context_lens, inv_freq, sink, heads, kv_rank, rot_dim, rot_dims, page_size,         \
                 num_pages, scale, window, cos_sin_scale)
  if (dtype == kFloat32) {
    if (kv_rank <= 512) LI_LATENT_LAUNCH(float, 16); else LI_LATENT_LAUNCH(float, 32);
  } else {
    if (kv_rank <= 512) LI_LATENT_LAUNCH(bf16, 16); else LI_LATENT_LAUNCH(bf16, 32);
  }
#undef LI_LATENT_LAUNCH
  return (int)e;
}

// out[t, h * vdim + e] = v[h, t, e] * sigmoid(gate[t * gate_stride + h * vdim + e]); gate null: v[h, t, e].
LI_EXPORT int li_gate_heads(int dtype, const void* v, const void* gate, int gate_stride, void* out, int tokens,
                            int heads, int vdim, cudaStream_t stream) {
  const size_t n = (size_t)tokens * heads * vdim;
  if (n == 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  cudaError_t e;
  if (dtype == kFloat32)
    e = launch_pdl(tokens, gate_heads_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)v,
                   (const float*)gate, gate_stride, (float*)out, tokens, heads, vdim);
  else
    e = launch_pdl(tokens, gate_heads_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)v,
                   (const bf16*)gate, gate_stride, (bf16*)out, tokens, heads, vdim);
  return (int)e;
}
