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
// three shuffles.  The tokens of a step come in chunks of 16: the block turns a chunk's q (scaled) and k into
// floats in shared memory once, one warp computes the chunk's gates a lane a token (the maxima by a scan whose
// elements are the maps m -> max(m + F, I)), and then the chain runs over the chunk.  Whole prompts, portions
// and single tokens run the same code from the state the step before left.  Sequences that bring no token touch
// nothing.
#include "common.cuh"

namespace li {

constexpr int kMlstmChunk = 16;
constexpr int kMlstmColumns = 16;   // per block: 128 threads, eight lanes a column

__device__ __forceinline__ float log_sigmoid(float z) {
  return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));
}

// NPL: entries of a column a lane keeps.  VEC: the lane's entries are float4 groups 4 * (sub + 8 j) .. + 3
// (dim a multiple of four, 16-byte aligned state); otherwise entries sub + 8 i.
template <typename T, int NPL, bool VEC>
__global__ void __launch_bounds__(128)
mlstm_kernel(const T* __restrict__ proj, size_t row_stride, int q_off, int k_off, int v_off, int i_off, int f_off,
             const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
             float* __restrict__ state, float* __restrict__ maxima, const int* __restrict__ query_start_loc,
             const int* __restrict__ state_slots, float* __restrict__ out, float* __restrict__ den, int heads, int dim,
             int vdim) {
  extern __shared__ __align__(16) float shared[];
  float* qs = shared;                              // [chunk][dim]
  float* ks = qs + kMlstmChunk * dim;              // [chunk][dim]
  float* vs = ks + kMlstmChunk * dim;              // [chunk][columns]
  float* as = vs + kMlstmChunk * kMlstmColumns;    // [chunk] decay of the state
  float* bs = as + kMlstmChunk;                    // [chunk] weight of the new token
  float* es = bs + kMlstmChunk;                    // [chunk] exp(-m)
  __shared__ float carried_max;

  const int seq = blockIdx.z, head = blockIdx.y;
  const int tid = threadIdx.x, sub = tid & 7, group = tid >> 3;
  const int begin = query_start_loc[seq], end = query_start_loc[seq + 1];
  if (end <= begin) return;
  const int slot = state_slots[seq];
  if (slot < 0) return;
  const int first_column = blockIdx.x * kMlstmColumns;
  const int column = first_column + group;
  const bool live = column <= vdim;
  const float scale = rsqrtf((float)dim);
  const float bias_i = i_bias[head], bias_f = f_bias[head];

  int at[NPL];            // which entry of the column register i holds; >= dim: none
#pragma unroll
  for (int i = 0; i < NPL; ++i) at[i] = VEC ? 4 * (sub + 8 * (i >> 2)) + (i & 3) : sub + 8 * i;

  grid_dependency_wait();
  float* mine = state + (((size_t)slot * heads + head) * (vdim + 1) + (live ? column : 0)) * dim;
  float* my_max = maxima + ((size_t)slot * heads + head) * (vdim + 1);
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
  if (tid == 0) carried_max = my_max[first_column];
  float m_last = 0.f;     // lane 0 of warp 0: the maximum after the newest token

  for (int t0 = begin; t0 < end; t0 += kMlstmChunk) {
    const int n = end - t0 < kMlstmChunk ? end - t0 : kMlstmChunk;
    __syncthreads();      // the chunk before is done with; carried_max is written
    for (int idx = tid; idx < n * dim; idx += 128) {
      const int tok = idx / dim, e = idx - tok * dim;
      const T* row = proj + (size_t)(t0 + tok) * row_stride + (size_t)head * dim + e;
      qs[idx] = to_float(row[q_off]) * scale;
      ks[idx] = to_float(row[k_off]);
    }
    for (int idx = tid; idx < n * kMlstmColumns; idx += 128) {
      const int tok = idx / kMlstmColumns, c = first_column + (idx - tok * kMlstmColumns);
      vs[idx] = c < vdim ? to_float(proj[(size_t)(t0 + tok) * row_stride + v_off + (size_t)head * vdim + c]) : 1.0f;
    }
    if (tid < 32) {
      // Gates of the chunk, a lane a token.  (F, I) stands for the map m -> max(m + F, I); a token's own map is
      // (f, i), and after the scan lane t holds the map of tokens 0..t of the chunk together.
      const bool has = tid < n;
      float gate_i = 0.f, gate_f = 0.f;
      if (has) {
        const T* row = proj + (size_t)(t0 + tid) * row_stride;
        gate_i = cap * tanhf((to_float(row[i_off + head]) + bias_i) / cap);
        gate_f = log_sigmoid(cap * tanhf((to_float(row[f_off + head]) + bias_f) / cap));
      }
      float F = gate_f, I = has ? gate_i : -INFINITY;
#pragma unroll
      for (int off = 1; off < kMlstmChunk; off <<= 1) {
        const float Fb = __shfl_up_sync(0xffffffffu, F, off), Ib = __shfl_up_sync(0xffffffffu, I, off);
        if (tid >= off) {
          I = fmaxf(Ib + F, I);
          F = Fb + F;
        }
      }
      const float m_in = carried_max;
      const float m = fmaxf(m_in + F, I);
      float m_before = __shfl_up_sync(0xffffffffu, m, 1);
      if (tid == 0) m_before = m_in;
      if (has) {
        as[tid] = expf(gate_f + m_before - m);
        bs[tid] = expf(gate_i - m);
        es[tid] = expf(-m);
      }
      m_last = __shfl_sync(0xffffffffu, m, n - 1);
      __syncwarp();
      if (tid == 0) carried_max = m_last;
    }
    __syncthreads();
    for (int tok = 0; tok < n; ++tok) {
      const float a = as[tok], bv = bs[tok] * vs[tok * kMlstmColumns + group];
      const float* q = qs + tok * dim;
      const float* k = ks + tok * dim;
      float part = 0.f;
      if (VEC) {
#pragma unroll
        for (int j = 0; j < NPL / 4; ++j) {
          if (at[4 * j] < dim) {
            const float4 kv = *reinterpret_cast<const float4*>(k + at[4 * j]);
            const float4 qv = *reinterpret_cast<const float4*>(q + at[4 * j]);
            S[4 * j] = fmaf(a, S[4 * j], bv * kv.x);
            S[4 * j + 1] = fmaf(a, S[4 * j + 1], bv * kv.y);
            S[4 * j + 2] = fmaf(a, S[4 * j + 2], bv * kv.z);
            S[4 * j + 3] = fmaf(a, S[4 * j + 3], bv * kv.w);
            part = fmaf(S[4 * j], qv.x, part);
            part = fmaf(S[4 * j + 1], qv.y, part);
            part = fmaf(S[4 * j + 2], qv.z, part);
            part = fmaf(S[4 * j + 3], qv.w, part);
          }
        }
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
  __syncthreads();
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
    if (sub == 0) my_max[column] = carried_max;
  }
}

template <typename T, int NPL, bool VEC>
int launch_mlstm(long tokens, dim3 grid, size_t smem, cudaStream_t stream, const void* proj, size_t row_stride,
                 int q_off, int k_off, int v_off, int i_off, int f_off, const float* i_bias, const float* f_bias,
                 float cap, float* state, float* maxima, const int* qsl, const int* slots, float* out, float* den,
                 int heads, int dim, int vdim) {
  return (int)launch_pdl(tokens, mlstm_kernel<T, NPL, VEC>, grid, dim3(128), smem, stream, (const T*)proj, row_stride,
                         q_off, k_off, v_off, i_off, f_off, i_bias, f_bias, cap, state, maxima, qsl, slots, out, den,
                         heads, dim, vdim);
}

template <typename T>
int dispatch_mlstm(int per_lane, bool vec, long tokens, dim3 grid, size_t smem, cudaStream_t stream, const void* proj,
                   size_t row_stride, int q_off, int k_off, int v_off, int i_off, int f_off, const float* i_bias,
                   const float* f_bias, float cap, float* state, float* maxima, const int* qsl, const int* slots,
                   float* out, float* den, int heads, int dim, int vdim) {
#define LI_MLSTM(NPL, VEC)                                                                                            \
  return launch_mlstm<T, NPL, VEC>(tokens, grid, smem, stream, proj, row_stride, q_off, k_off, v_off, i_off, f_off,   \
                                   i_bias, f_bias, cap, state, maxima, qsl, slots, out, den, heads, dim, vdim)
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
}

}  // namespace li

using namespace li;

// proj [tokens, row_stride]: per token the heads' q (at column q_off, heads x dim), k (k_off), v (v_off, heads x
// vdim) and the raw gates (i_off, f_off: one per head).  state [slots, heads, vdim + 1, dim] and maxima
// [slots, heads, vdim + 1] float32 are read and written; out [tokens, heads * vdim] and den [tokens, heads] float32.
LI_EXPORT int li_mlstm(int dtype, const void* proj, size_t row_stride, int q_off, int k_off, int v_off, int i_off,
                       int f_off, const float* i_bias, const float* f_bias, float cap, float* state, float* maxima,
                       const int* query_start_loc, const int* state_slots, int tokens, int num_seqs, float* out,
                       float* den, int heads, int dim, int vdim, cudaStream_t stream) {
  if (tokens <= 0 || num_seqs <= 0) return 0;
  if (heads < 1 || heads > 65535 || num_seqs > 65535 || dim < 1 || dim > 256 || vdim < 1 || !(cap > 0.f))
    return LI_ERR_UNSUPPORTED;
  const dim3 grid((vdim + 1 + kMlstmColumns - 1) / kMlstmColumns, heads, num_seqs);
  const size_t smem = ((size_t)2 * kMlstmChunk * dim + kMlstmChunk * kMlstmColumns + 3 * kMlstmChunk) * sizeof(float);
  const bool vec = dim % 4 == 0 && aligned16(state);
  const int per_lane = vec ? 4 * ((dim / 4 + 7) / 8) : (dim + 7) / 8;
  if (dtype == kFloat32)
    return dispatch_mlstm<float>(per_lane, vec, tokens, grid, smem, stream, proj, row_stride, q_off, k_off, v_off, i_off,
                                 f_off, i_bias, f_bias, cap, state, maxima, query_start_loc, state_slots, out, den,
                                 heads, dim, vdim);
  return dispatch_mlstm<bf16>(per_lane, vec, tokens, grid, smem, stream, proj, row_stride, q_off, k_off, v_off, i_off,
                              f_off, i_bias, f_bias, cap, state, maxima, query_start_loc, state_slots, out, den, heads,
                              dim, vdim);
}
