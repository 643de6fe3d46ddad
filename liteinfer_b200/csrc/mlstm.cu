// The matrix memory of an mLSTM layer: per request and head a state S [dim, vdim] and a normaliser n [dim] in
// 32-bit, kept stable by a running maximum m of the gates' logarithms.
//
//   li_mlstm   per token, with raw gate inputs x_i, x_f of the head (bias added, then capped):
//                  i = cap * tanh(x_i / cap);  f = logsigmoid(cap * tanh(x_f / cap))
//                  m' = max(f + m, i);  a = exp(f + m - m');  b = exp(i - m')
//                  S <- a S + b k v^T;  n <- a n + b k;  m <- m'
//                  o = S^T (q * dim^-0.5);  den = max(|n . q * dim^-0.5|, exp(-m)) + 1e-6
//              The read-out is written unnormalised, den beside it; the norm behind this kernel divides.
//
// n obeys the recurrence of a column of S whose value is always 1, so the kernel runs vdim + 1 columns: the
// state is kept column by column, state[slot][head][vdim + 1][dim] with n as the last column, and every
// column is a chain of its own over the tokens.  Each column also keeps its own copy of m
// (maxima[slot][head][vdim + 1]): a block reads and writes only its own columns, so blocks of one head need
// no order among themselves.  A block takes 16 columns of one head of one sequence; eight lanes share a column,
// each with dim/8 of its entries in registers for the whole step, and add up their parts of the read-out with
// three shuffles.  The tokens of a step come in chunks (16 tokens, 8 for wide heads).  A fifth warp works one
// chunk ahead of the four that run the chain: it turns the chunk's q (scaled), k and the block's columns of v
// into floats in shared memory, 16 bytes a load and several loads in flight, and computes the chunk's gates a
// lane a token (the maxima by a scan whose elements are the maps m -> max(m + F, I)); the running maximum
// stays in its registers from chunk to chunk.  Two buffers and one block-wide barrier a chunk.  Whole prompts,
// portions and single tokens run the same code from the state the step before left.  Sequences that bring no
// token touch nothing.
#include "common.cuh"

namespace li {

constexpr int kMlstmColumns = 16;   // per block: 128 chain threads, eight lanes a column
constexpr int kMlstmThreads = 160;  // and the warp that prepares the next chunk

__device__ __forceinline__ float log_sigmoid(float z) {
  return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));
}

// One chunk's inputs into a buffer: q [chunk][dim] (scaled), k [chunk][dim], v [chunk][16] (1 from column vdim
// on).  vec: every source vector of 16 bytes is aligned and lies within one of q, k, v.  U: loads a lane has in
// flight at once; they are the preparing warp's registers, and the kernel's register count is the larger of
// the two roles', so a step of single tokens, which has little to stage and lives on many blocks a
// multiprocessor, takes U = 1.
template <typename T, int U>
__device__ __forceinline__ void mlstm_fill(float* qs, float* ks, float* vs, const T* __restrict__ proj,
                                           size_t row_stride, int q_at, int k_at, int v_at, int first_column, int t0,
                                           int n, int dim, int vdim, float scale, bool vec, int lane) {
  if (vec) {
    constexpr int N = Vec16<T>::N;
    const int dv = dim / N, cv = kMlstmColumns / N, per_tok = 2 * dv + cv;
    const int items = n * per_tok;
    for (int base = 0; base < items; base += 32 * U) {
      Vec16<T> raw[U];
      int where[U];      // destination in floats from qs; -1: nothing
      float factor[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = base + u * 32 + lane;
        where[u] = -1;
        if (idx < items) {
          const int tok = idx / per_tok, r = idx - tok * per_tok;
          const T* row = proj + (size_t)(t0 + tok) * row_stride;
          if (r < dv) {
            raw[u] = load16(row + q_at + r * N);
            where[u] = tok * dim + r * N;
            factor[u] = scale;
          } else if (r < 2 * dv) {
            raw[u] = load16(row + k_at + (r - dv) * N);
            where[u] = (int)(ks - qs) + tok * dim + (r - dv) * N;
            factor[u] = 1.0f;
          } else {
            const int c = (r - 2 * dv) * N;
            where[u] = (int)(vs - qs) + tok * kMlstmColumns + c;
            if (first_column + c < vdim) {
              raw[u] = load16(row + v_at + first_column + c);
              factor[u] = 1.0f;
            } else {
              factor[u] = 0.f;   // columns past the values: the normaliser's 1
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (where[u] < 0) continue;
        float x[N];
        if (factor[u] == 0.f) {
#pragma unroll
          for (int e = 0; e < N; ++e) x[e] = 1.0f;
        } else {
          unpack16(raw[u], x);
#pragma unroll
          for (int e = 0; e < N; ++e) x[e] *= factor[u];
        }
        float* dst = qs + where[u];
#pragma unroll
        for (int e = 0; e < N; e += 4) *reinterpret_cast<float4*>(dst + e) = make_float4(x[e], x[e + 1], x[e + 2], x[e + 3]);
      }
    }
    return;
  }
  for (int idx = lane; idx < n * dim; idx += 32) {
    const int tok = idx / dim, e = idx - tok * dim;
    const T* row = proj + (size_t)(t0 + tok) * row_stride + e;
    qs[idx] = to_float(row[q_at]) * scale;
    ks[idx] = to_float(row[k_at]);
  }
  for (int idx = lane; idx < n * kMlstmColumns; idx += 32) {
    const int tok = idx / kMlstmColumns, c = first_column + (idx - tok * kMlstmColumns);
    vs[idx] = c < vdim ? to_float(proj[(size_t)(t0 + tok) * row_stride + v_at + c]) : 1.0f;
  }
}

// NPL: entries of a column a lane keeps.  VEC: the lane's entries are float4 groups 4 * (sub + 8 j) .. + 3
// (dim a multiple of four, 16-byte aligned state); otherwise entries sub + 8 i.
template <typename T, int NPL, bool VEC, int U>
__global__ void __launch_bounds__(kMlstmThreads)
mlstm_kernel(const T* __restrict__ proj, size_t row_stride, int q_off, int k_off, int v_off, int i_off, int f_off,
             const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
             float* __restrict__ state, float* __restrict__ maxima, const int* __restrict__ query_start_loc,
             const int* __restrict__ state_slots, float* __restrict__ out, float* __restrict__ den, int heads, int dim,
             int vdim, int chunk, int vec_in) {
  extern __shared__ __align__(16) float shared[];
  // A buffer: q [chunk][dim], k [chunk][dim], v [chunk][columns], then per token the state's decay, the new
  // token's weight and exp(-m).
  const int per_buffer = chunk * (2 * dim + kMlstmColumns + 3);

  const int seq = blockIdx.z, head = blockIdx.y;
  const int tid = threadIdx.x;
  const int begin = query_start_loc[seq], end = query_start_loc[seq + 1];
  if (end <= begin) return;
  const int slot = state_slots[seq];
  if (slot < 0) return;
  const int first_column = blockIdx.x * kMlstmColumns;
  const int chunks = (end - begin + chunk - 1) / chunk;
  float* my_max = maxima + ((size_t)slot * heads + head) * (vdim + 1);

  if (tid >= 128) {
    // ---- the warp that prepares: inputs and gates of chunk c + 1 while the chain runs over chunk c
    const int lane = tid - 128;
    const float scale = rsqrtf((float)dim);
    const float bias_i = i_bias[head], bias_f = f_bias[head];
    grid_dependency_wait();
    float m_run = my_max[first_column];
    for (int c = 0; c <= chunks; ++c) {
      if (c < chunks) {
        const int t0 = begin + c * chunk;
        const int n = end - t0 < chunk ? end - t0 : chunk;
        float* qs = shared + (c & 1) * per_buffer;
        float* ks = qs + chunk * dim;
        float* vs = ks + chunk * dim;
        float* as = vs + chunk * kMlstmColumns;
        float* bs = as + chunk;
        float* es = bs + chunk;
        // Gates, a lane a token.  (F, I) stands for the map m -> max(m + F, I); a token's own map is (f, i), and
        // after the scan lane t holds the map of tokens 0..t of the chunk together.
        const bool has = lane < n;
        float gate_i = 0.f, gate_f = 0.f;
        if (has) {
          const T* row = proj + (size_t)(t0 + lane) * row_stride;
          gate_i = cap * tanhf((to_float(row[i_off + head]) + bias_i) / cap);
          gate_f = log_sigmoid(cap * tanhf((to_float(row[f_off + head]) + bias_f) / cap));
        }
        mlstm_fill<T, U>(qs, ks, vs, proj, row_stride, q_off + head * dim, k_off + head * dim, v_off + head * vdim,
                      first_column, t0, n, dim, vdim, scale, vec_in != 0, lane);
        float F = gate_f, I = has ? gate_i : -INFINITY;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const float Fb = __shfl_up_sync(0xffffffffu, F, off), Ib = __shfl_up_sync(0xffffffffu, I, off);
          if (lane >= off) {
            I = fmaxf(Ib + F, I);
            F = Fb + F;
          }
        }
        const float m = fmaxf(m_run + F, I);
        float m_before = __shfl_up_sync(0xffffffffu, m, 1);
        if (lane == 0) m_before = m_run;
        if (has) {
          as[lane] = expf(gate_f + m_before - m);
          bs[lane] = expf(gate_i - m);
          es[lane] = expf(-m);
        }
        m_run = __shfl_sync(0xffffffffu, m, n - 1);
      }
      __syncthreads();     // chunk c is ready; the chain is done with chunk c - 1
    }
    const int column = first_column + lane;
    if (lane < kMlstmColumns && column <= vdim) my_max[column] = m_run;
    return;
  }

  // ---- the chain
  const int sub = tid & 7, group = tid >> 3;
  const int column = first_column + group;
  const bool live = column <= vdim;
  int at[NPL];            // which entry of the column register i holds; >= dim: none
#pragma unroll
  for (int i = 0; i < NPL; ++i) at[i] = VEC ? 4 * (sub + 8 * (i >> 2)) + (i & 3) : sub + 8 * i;

  grid_dependency_wait();
  float* mine = state + (((size_t)slot * heads + head) * (vdim + 1) + (live ? column : 0)) * dim;
  float S[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) S[i] = 0.f;
  if (live) {
    if (VEC) {
#pragma unroll
      for (int j = 0; j < NPL / 4; ++j)
        if (at[4 * j] < dim) {
          const float4 v = *reinterpret_cast<const float4*>(mine + at[4 * j]);
          S[4 * j] = v.x; S[4 * j + 1] = v.y; S[4 * j + 2] = v.z; S[4 * j + 3] = v.w;
        }
    } else {
#pragma unroll
      for (int i = 0; i < NPL; ++i)
        if (at[i] < dim) S[i] = mine[at[i]];
    }
  }

  for (int c = 0; c < chunks; ++c) {
    __syncthreads();      // chunk c is ready
    const int t0 = begin + c * chunk;
    const int n = end - t0 < chunk ? end - t0 : chunk;
    const float* qs = shared + (c & 1) * per_buffer;
    const float* ks = qs + chunk * dim;
    const float* vs = ks + chunk * dim;
    const float* as = vs + chunk * kMlstmColumns;
    const float* bs = as + chunk;
    const float* es = bs + chunk;
    for (int tok = 0; tok < n; ++tok) {
      const float a = as[tok], bv = bs[tok] * vs[tok * kMlstmColumns + group];
      const float* q = qs + tok * dim;
      const float* k = ks + tok * dim;
      float part = 0.f;
      if (VEC) {
        float parts[NPL / 4 > 0 ? NPL / 4 : 1];   // a partial sum per group of four: short chains of additions
#pragma unroll
        for (int j = 0; j < NPL / 4; ++j) {
          parts[j] = 0.f;
          if (at[4 * j] < dim) {
            const float4 kv = *reinterpret_cast<const float4*>(k + at[4 * j]);
            const float4 qv = *reinterpret_cast<const float4*>(q + at[4 * j]);
            S[4 * j] = fmaf(a, S[4 * j], bv * kv.x);
            S[4 * j + 1] = fmaf(a, S[4 * j + 1], bv * kv.y);
            S[4 * j + 2] = fmaf(a, S[4 * j + 2], bv * kv.z);
            S[4 * j + 3] = fmaf(a, S[4 * j + 3], bv * kv.w);
            parts[j] = fmaf(S[4 * j + 3], qv.w, fmaf(S[4 * j + 2], qv.z, fmaf(S[4 * j + 1], qv.y, S[4 * j] * qv.x)));
          }
        }
#pragma unroll
        for (int j = 0; j < NPL / 4; ++j) part += parts[j];
      } else {
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          if (at[i] < dim) {
            S[i] = fmaf(a, S[i], bv * k[at[i]]);
            part = fmaf(S[i], q[at[i]], part);
          }
        }
      }
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      if (sub == 0 && live) {
        if (column < vdim) out[(size_t)(t0 + tok) * heads * vdim + (size_t)head * vdim + column] = part;
        else den[(size_t)(t0 + tok) * heads + head] = fmaxf(fabsf(part), es[tok]) + 1e-6f;
      }
    }
  }
  __syncthreads();        // the preparing warp's last barrier
  if (live) {
    if (VEC) {
#pragma unroll
      for (int j = 0; j < NPL / 4; ++j)
        if (at[4 * j] < dim)
          *reinterpret_cast<float4*>(mine + at[4 * j]) = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < NPL; ++i)
        if (at[i] < dim) mine[at[i]] = S[i];
    }
  }
}

template <typename T, int NPL, bool VEC, int U>
int launch_mlstm(long tokens, dim3 grid, size_t smem, cudaStream_t stream, const void* proj, size_t row_stride,
                 int q_off, int k_off, int v_off, int i_off, int f_off, const float* i_bias, const float* f_bias,
                 float cap, float* state, float* maxima, const int* qsl, const int* slots, float* out, float* den,
                 int heads, int dim, int vdim, int chunk, int vec_in) {
  return (int)launch_pdl(tokens, mlstm_kernel<T, NPL, VEC, U>, grid, dim3(kMlstmThreads), smem, stream, (const T*)proj,
                         row_stride, q_off, k_off, v_off, i_off, f_off, i_bias, f_bias, cap, state, maxima, qsl, slots,
                         out, den, heads, dim, vdim, chunk, vec_in);
}

template <typename T>
int dispatch_mlstm(int per_lane, bool vec, long tokens, dim3 grid, size_t smem, cudaStream_t stream, const void* proj,
                   size_t row_stride, int q_off, int k_off, int v_off, int i_off, int f_off, const float* i_bias,
                   const float* f_bias, float cap, float* state, float* maxima, const int* qsl, const int* slots,
                   float* out, float* den, int heads, int dim, int vdim, int chunk) {
  // The preparing warp loads 16 bytes at a time where every such vector is aligned and lies within q, k or v.
  constexpr int N = Vec16<T>::N;
  const int vec_in = dim % N == 0 && vdim % N == 0 && row_stride % N == 0 && q_off % N == 0 && k_off % N == 0 &&
                     v_off % N == 0 && aligned16(proj);
#define LI_MLSTM_U(NPL, VEC, U)                                                                                       \
  return launch_mlstm<T, NPL, VEC, U>(tokens, grid, smem, stream, proj, row_stride, q_off, k_off, v_off, i_off, f_off, \
                                      i_bias, f_bias, cap, state, maxima, qsl, slots, out, den, heads, dim, vdim,      \
                                      chunk, vec_in)
#define LI_MLSTM(NPL, VEC)                                                                                            \
  {                                                                                                                   \
    if (chunk == 1) LI_MLSTM_U(NPL, VEC, 1);                                                                          \
    LI_MLSTM_U(NPL, VEC, 8);                                                                                          \
  }
  if (vec) {
    if (per_lane <= 4) LI_MLSTM(4, true);
    if (per_lane <= 8) LI_MLSTM(8, true);
    if (per_lane <= 16) LI_MLSTM(16, true);
    LI_MLSTM(32, true);
  }
  if (per_lane <= 1) LI_MLSTM(1, false);
  if (per_lane <= 2) LI_MLSTM(2, false);
  if (per_lane <= 4) LI_MLSTM(4, false);
  if (per_lane <= 8) LI_MLSTM(8, false);
  if (per_lane <= 16) LI_MLSTM(16, false);
  LI_MLSTM(32, false);
#undef LI_MLSTM
#undef LI_MLSTM_U
}

}  // namespace li

using namespace li;

// proj [tokens, row_stride]: per token the heads' q (at column q_off, heads x dim), k (k_off), v (v_off, heads x
// vdim) and the raw gates (i_off, f_off: one per head).  state [slots, heads, vdim + 1, dim] and maxima
// [slots, heads, vdim + 1] float32 are read and written; out [tokens, heads * vdim] and den [tokens, heads] float32.
LI_EXPORT int li_mlstm(int dtype, const void* proj, size_t row_stride, int q_off, int k_off, int v_off, int i_off,
                       int f_off, const float* i_bias, const float* f_bias, float cap, float* state, float* maxima,
                       const int* query_start_loc, const int* state_slots, int tokens, int num_seqs, float* out,
                       float* den, int heads, int dim, int vdim, int max_query_len, cudaStream_t stream) {
  if (tokens <= 0 || num_seqs <= 0) return 0;
  if (heads < 1 || heads > 65535 || num_seqs > 65535 || dim < 1 || dim > 256 || vdim < 1 || !(cap > 0.f))
    return LI_ERR_UNSUPPORTED;
  const dim3 grid((vdim + 1 + kMlstmColumns - 1) / kMlstmColumns, heads, num_seqs);
  // Two buffers within 48 KB; no longer than the longest sequence of the step where the caller knows it, so that
  // a step of single tokens keeps many blocks on a multiprocessor and their state loads in flight.
  int chunk = dim <= 160 ? 16 : 8;
  if (max_query_len > 0 && max_query_len < chunk) chunk = max_query_len;
  const size_t smem = (size_t)2 * chunk * (2 * dim + kMlstmColumns + 3) * sizeof(float);
  const bool vec = dim % 4 == 0 && aligned16(state);
  const int per_lane = vec ? 4 * ((dim / 4 + 7) / 8) : (dim + 7) / 8;
  if (dtype == kFloat32)
    return dispatch_mlstm<float>(per_lane, vec, tokens, grid, smem, stream, proj, row_stride, q_off, k_off, v_off, i_off,
                                 f_off, i_bias, f_bias, cap, state, maxima, query_start_loc, state_slots, out, den,
                                 heads, dim, vdim, chunk);
  return dispatch_mlstm<bf16>(per_lane, vec, tokens, grid, smem, stream, proj, row_stride, q_off, k_off, v_off, i_off,
                              f_off, i_bias, f_bias, cap, state, maxima, query_start_loc, state_slots, out, den, heads,
                              dim, vdim, chunk);
}
