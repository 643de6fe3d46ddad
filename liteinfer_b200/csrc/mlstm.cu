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
// each with dim/8 of its entries in registers for the whole step.  The tokens of a step come in chunks (16
// tokens, 8 for wide heads).  Warps beside the four that run the chain work one chunk ahead of them: they turn
// the chunk's q (scaled), k and the block's columns of v into floats in shared memory, 16 bytes a load and all
// loads of a chunk in flight at once, and the first of them computes the chunk's gates a lane a token (the
// maxima by a scan whose elements are the maps m -> max(m + F, I)); the running maximum stays in its registers
// from chunk to chunk.  Two buffers and one block-wide barrier a chunk.  A token's update of S needs nothing of
// its read-out, so the chain keeps the lanes' parts of eight tokens' read-outs and adds them up together.  Whole
// prompts, portions and single tokens run the same code from the state the step before left (in a step of single
// tokens the chain's threads fetch their token themselves and the fifth warp has only the gates), and a read-out
// is the same sum in the same order wherever its token stands in a step.  Sequences that bring no token touch
// nothing.
#include "common.cuh"

namespace li {

constexpr int kMlstmColumns = 16;   // per block: 128 chain threads, eight lanes a column
constexpr int kMlstmThreads = 256;  // and up to four warps that prepare the next chunk (one for single tokens)

__device__ __forceinline__ float log_sigmoid(float z) {
  return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));
}

// One chunk's inputs into a buffer: q [chunk][dimp] (scaled), k [chunk][dimp], v [chunk][16] (1 from column vdim
// on); the entries dim .. dimp - 1 of a row are left alone.  vec: every source vector of 16 bytes is aligned and
// lies within one of q, k, v.  U: loads a lane has in flight at once; they are the preparing warp's registers, and the kernel's register count is the larger of
// the two roles', so a step of single tokens, which has little to stage and lives on many blocks a
// multiprocessor, takes U = 1.
template <typename T, int U>
__device__ __forceinline__ void mlstm_fill(float* qs, float* ks, float* vs, const T* __restrict__ proj,
                                           size_t row_stride, int q_at, int k_at, int v_at, int first_column, int t0,
                                           int n, int dim, int dimp, int vdim, float scale, bool vec, int who, int team) {
  if (vec) {
    constexpr int N = Vec16<T>::N;
    const int dv = dim / N, cv = kMlstmColumns / N, per_tok = 2 * dv + cv;
    const int items = n * per_tok;
    // Every load of a round is issued whatever its lane's item is (the address is made by selection, an item
    // past the end or past the values reads a valid place and is discarded), so that U loads a lane are in
    // flight together.
    for (int base = 0; base < items; base += team * U) {
      Vec16<T> raw[U];
      int where[U];      // destination in floats from qs; -1: nothing
      float factor[U];   // 0: columns past the values, the normaliser's 1
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = base + u * team + who;
        const bool valid = idx < items;
        const int tok = valid ? idx / per_tok : 0, r = valid ? idx - tok * per_tok : 0;
        const bool is_q = r < dv, is_k = !is_q && r < 2 * dv;
        const int c = (r - 2 * dv) * N;                       // the value's column within the block
        const bool is_one = !is_q && !is_k && first_column + c >= vdim;
        const int column = is_q ? q_at + r * N : is_k ? k_at + (r - dv) * N : is_one ? v_at : v_at + first_column + c;
        raw[u] = load16(proj + (size_t)(t0 + tok) * row_stride + column);
        where[u] = !valid ? -1
                   : is_q ? tok * dimp + r * N
                   : is_k ? (int)(ks - qs) + tok * dimp + (r - dv) * N
                          : (int)(vs - qs) + tok * kMlstmColumns + c;
        factor[u] = is_q ? scale : is_one ? 0.f : 1.0f;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (where[u] < 0) continue;
        float x[N];
        unpack16(raw[u], x);
#pragma unroll
        for (int e = 0; e < N; ++e) x[e] = factor[u] == 0.f ? 1.0f : x[e] * factor[u];
        float* dst = qs + where[u];
#pragma unroll
        for (int e = 0; e < N; e += 4) *reinterpret_cast<float4*>(dst + e) = make_float4(x[e], x[e + 1], x[e + 2], x[e + 3]);
      }
    }
    return;
  }
  for (int idx = who; idx < n * dim; idx += team) {
    const int tok = idx / dim, e = idx - tok * dim;
    const T* row = proj + (size_t)(t0 + tok) * row_stride + e;
    qs[tok * dimp + e] = to_float(row[q_at]) * scale;
    ks[tok * dimp + e] = to_float(row[k_at]);
  }
  for (int idx = who; idx < n * kMlstmColumns; idx += team) {
    const int tok = idx / kMlstmColumns, c = first_column + (idx - tok * kMlstmColumns);
    vs[idx] = c < vdim ? to_float(proj[(size_t)(t0 + tok) * row_stride + v_at + c]) : 1.0f;
  }
}

// One token on a lane's part of a column: S <- a S + bv k, and the lane's part of S . q.  q and k point at the
// token's rows of 8 NPL floats in shared memory.
template <int NPL, bool VEC>
__device__ __forceinline__ float mlstm_token(float (&S)[NPL], const float* __restrict__ q, const float* __restrict__ k,
                                             float a, float bv, int sub) {
  float part = 0.f;
  if (VEC) {
    float parts[NPL / 4 > 0 ? NPL / 4 : 1];   // a partial sum per group of four: short chains of additions
#pragma unroll
    for (int j = 0; j < NPL / 4; ++j) {
      const float4 kv = *reinterpret_cast<const float4*>(k + 4 * (sub + 8 * j));
      const float4 qv = *reinterpret_cast<const float4*>(q + 4 * (sub + 8 * j));
      S[4 * j] = fmaf(a, S[4 * j], bv * kv.x);
      S[4 * j + 1] = fmaf(a, S[4 * j + 1], bv * kv.y);
      S[4 * j + 2] = fmaf(a, S[4 * j + 2], bv * kv.z);
      S[4 * j + 3] = fmaf(a, S[4 * j + 3], bv * kv.w);
      parts[j] = fmaf(S[4 * j + 3], qv.w, fmaf(S[4 * j + 2], qv.z, fmaf(S[4 * j + 1], qv.y, S[4 * j] * qv.x)));
    }
#pragma unroll
    for (int j = 0; j < NPL / 4; ++j) part += parts[j];
  } else {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      S[i] = fmaf(a, S[i], bv * k[sub + 8 * i]);
      part = fmaf(S[i], q[sub + 8 * i], part);
    }
  }
  return part;
}

// NPL: entries of a column a lane keeps.  VEC: the lane's entries are float4 groups 4 * (sub + 8 j) .. + 3
// (dim a multiple of four, 16-byte aligned state); otherwise entries sub + 8 i.
template <typename T, int NPL, bool VEC, int U>
__global__ void __launch_bounds__(U == 1 ? 160 : kMlstmThreads, U == 1 && NPL <= 16 ? 6 : (NPL <= 16 ? 3 : 2))
mlstm_kernel(const T* __restrict__ proj, size_t row_stride, int q_off, int k_off, int v_off, int i_off, int f_off,
             const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
             float* __restrict__ state, float* __restrict__ maxima, const int* __restrict__ query_start_loc,
             const int* __restrict__ state_slots, float* __restrict__ out, float* __restrict__ den, int heads, int dim,
             int vdim, int chunk, int vec_in) {
  extern __shared__ __align__(16) float shared[];
  // A buffer: q [chunk][dimp], k [chunk][dimp], v [chunk][columns], then per token the state's decay, the new
  // token's weight and exp(-m).  dimp = 8 NPL: a row has a place for every register of the chain's lanes, and
  // the places past dim hold zeros, so the chain runs without asking which of its registers are in use.
  constexpr int dimp = 8 * NPL;
  const int per_buffer = chunk * (2 * dimp + kMlstmColumns + 3);

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
    // ---- the warps that prepare: inputs and gates of chunk c + 1 while the chain runs over chunk c.  All of
    // them stage q, k and v; the first also computes the gates, a lane a token.
    const int who = tid - 128, team = (int)blockDim.x - 128, lane = who & 31;
    const bool gates = who < 32;
    const float scale = rsqrtf((float)dim);
    const float bias_i = i_bias[head], bias_f = f_bias[head];
    if (dim < dimp)
      for (int idx = who; idx < 4 * chunk * (dimp - dim); idx += team) {
        const int row = idx / (dimp - dim), e = dim + idx - row * (dimp - dim);      // rows: buffer, q or k, token
        shared[(row / (2 * chunk)) * per_buffer + (row % (2 * chunk)) * dimp + e] = 0.f;
      }
    grid_dependency_wait();
    float m_run = gates ? my_max[first_column] : 0.f;
    for (int c = 0; c <= chunks; ++c) {
      if (c < chunks) {
        const int t0 = begin + c * chunk;
        const int n = end - t0 < chunk ? end - t0 : chunk;
        float* qs = shared + (c & 1) * per_buffer;
        float* ks = qs + chunk * dimp;
        float* vs = ks + chunk * dimp;
        float* as = vs + chunk * kMlstmColumns;
        float* bs = as + chunk;
        float* es = bs + chunk;
        // Gates.  (F, I) stands for the map m -> max(m + F, I); a token's own map is (f, i), and after the scan
        // lane t holds the map of tokens 0..t of the chunk together.
        const bool has = gates && lane < n;
        float raw_i = 0.f, raw_f = 0.f;
        if (has) {
          const T* row = proj + (size_t)(t0 + lane) * row_stride;
          raw_i = to_float(row[i_off + head]);
          raw_f = to_float(row[f_off + head]);
        }
        if (U > 1)
          mlstm_fill<T, U>(qs, ks, vs, proj, row_stride, q_off + head * dim, k_off + head * dim, v_off + head * vdim,
                           first_column, t0, n, dim, dimp, vdim, scale, vec_in != 0, who, team);
        if (gates) {
          const float gate_i = has ? cap * tanhf((raw_i + bias_i) / cap) : 0.f;
          const float gate_f = has ? log_sigmoid(cap * tanhf((raw_f + bias_f) / cap)) : 0.f;
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
      }
      __syncthreads();     // chunk c is ready; the chain is done with chunk c - 1
    }
    const int column = first_column + lane;
    if (gates && lane < kMlstmColumns && column <= vdim) my_max[column] = m_run;
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

  // Where this column writes: one read-out a token, or the divisor if it is the normaliser's column.
  const bool is_den = column == vdim;
  const size_t out_step = is_den ? (size_t)heads : (size_t)heads * vdim;
  float* target = is_den ? den + (size_t)begin * heads + head
                         : out + (size_t)begin * heads * vdim + (size_t)head * vdim + (live ? column : 0);

  for (int c = 0; c < chunks; ++c) {
    const int t0 = begin + c * chunk;
    const int n = end - t0 < chunk ? end - t0 : chunk;
    if (U == 1) {
      // Chunks of one (a step of single tokens): the chain's own threads fetch the token, beside their loads of
      // the state, while the fifth warp computes its gates.
      float* qw = shared + (c & 1) * per_buffer;
      mlstm_fill<T, 1>(qw, qw + chunk * dimp, qw + 2 * chunk * dimp, proj, row_stride, q_off + head * dim,
                       k_off + head * dim, v_off + head * vdim, first_column, t0, n, dim, dimp, vdim,
                       rsqrtf((float)dim), vec_in != 0, tid, 128);
    }
    __syncthreads();      // chunk c is ready
    const float* qs = shared + (c & 1) * per_buffer;
    const float* ks = qs + chunk * dimp;
    const float* vs = ks + chunk * dimp + group;
    const float* as = vs - group + chunk * kMlstmColumns;
    const float* bs = as + chunk;
    const float* es = bs + chunk;
    // A token's update of S needs only S; its read-out hangs off the side.  The eight lanes of a column keep
    // their parts of eight tokens' read-outs and add them up together: lane s ends with the sum of token s,
    // seven shuffles for eight tokens, and in between the chain runs undisturbed.  Every sum is the tree
    // ((s, s^4), (s^2, s^6)), ((s^1, s^5), (s^3, s^7)) whatever the token's place, so the cut changes no bit.
    for (int g0 = 0; g0 < n; g0 += 8) {
      float p[8];
      if (U > 1 && n - g0 >= 8) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          p[i] = mlstm_token<NPL, VEC>(S, qs + (g0 + i) * dimp, ks + (g0 + i) * dimp, as[g0 + i],
                                       bs[g0 + i] * vs[(g0 + i) * kMlstmColumns], sub);
      } else {
#pragma unroll
        for (int i = 0; i < (U > 1 ? 8 : 1); ++i) {
          p[i] = 0.f;
          if (g0 + i < n)
            p[i] = mlstm_token<NPL, VEC>(S, qs + (g0 + i) * dimp, ks + (g0 + i) * dimp, as[g0 + i],
                                         bs[g0 + i] * vs[(g0 + i) * kMlstmColumns], sub);
        }
      }
      float mine_sum;
      int mine_tok;
      if (U > 1) {
        float h[4], d[2];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const bool up = (sub & 4) != 0;
          h[i] = (up ? p[i + 4] : p[i]) + __shfl_xor_sync(0xffffffffu, up ? p[i] : p[i + 4], 4);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const bool up = (sub & 2) != 0;
          d[i] = (up ? h[i + 2] : h[i]) + __shfl_xor_sync(0xffffffffu, up ? h[i] : h[i + 2], 2);
        }
        const bool up = (sub & 1) != 0;
        mine_sum = (up ? d[1] : d[0]) + __shfl_xor_sync(0xffffffffu, up ? d[0] : d[1], 1);
        mine_tok = g0 + sub;
      } else {
        mine_sum = p[0];
        mine_sum += __shfl_xor_sync(0xffffffffu, mine_sum, 4);
        mine_sum += __shfl_xor_sync(0xffffffffu, mine_sum, 2);
        mine_sum += __shfl_xor_sync(0xffffffffu, mine_sum, 1);
        mine_tok = sub == 0 ? g0 : n;
      }
      if (live && mine_tok < n)
        target[(size_t)(c * chunk + mine_tok) * out_step] = is_den ? fmaxf(fabsf(mine_sum), es[mine_tok]) + 1e-6f : mine_sum;
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
  return (int)launch_pdl(tokens, mlstm_kernel<T, NPL, VEC, U>, grid, dim3(U == 1 ? 160 : kMlstmThreads), smem, stream, (const T*)proj,
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
    LI_MLSTM_U(NPL, VEC, 5);                                                                                          \
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
  const bool vec = dim % 4 == 0 && aligned16(state);
  // Registers a lane of the chain keeps of its column: the variant the dispatch below picks.
  int per_lane = vec ? 4 : 1;
  while (per_lane * 8 < dim) per_lane *= 2;
  const int dimp = 8 * per_lane;
  // Two buffers within 48 KB; no longer than the longest sequence of the step where the caller knows it, so that
  // a step of single tokens keeps many blocks on a multiprocessor and their state loads in flight.
  int chunk = dimp <= 160 ? 16 : 8;
  if (max_query_len > 0 && max_query_len < chunk) chunk = max_query_len;
  const size_t smem = (size_t)2 * chunk * (2 * dimp + kMlstmColumns + 3) * sizeof(float);
  if (dtype == kFloat32)
    return dispatch_mlstm<float>(per_lane, vec, tokens, grid, smem, stream, proj, row_stride, q_off, k_off, v_off, i_off,
                                 f_off, i_bias, f_bias, cap, state, maxima, query_start_loc, state_slots, out, den,
                                 heads, dim, vdim, chunk);
  return dispatch_mlstm<bf16>(per_lane, vec, tokens, grid, smem, stream, proj, row_stride, q_off, k_off, v_off, i_off,
                              f_off, i_bias, f_bias, cap, state, maxima, query_start_loc, state_slots, out, den, heads,
                              dim, vdim, chunk);
}
