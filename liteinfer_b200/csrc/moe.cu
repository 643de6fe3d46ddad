// A mixture of experts: routing, and the experts' products grouped by expert.
//
//   li_moe_route     per token: scores = softmax over all experts of the router's logits (32-bit); where the experts
//                    form `groups` equal groups of neighbours, a group's score is its largest score and only experts
//                    of the best `keep` groups can be chosen; the `top` largest scores among those are chosen (ties
//                    go to the lower index); the weights are the chosen scores, or those divided by their sum.
//   li_moe_sort      the (token, slot) pairs ordered by expert, each expert's run cut into tiles of `tile_rows` rows:
//                    order[], offsets[experts + 1], and per tile its expert and first row (-1: no such tile).
//   li_moe_grouped   out[pair] = f(W_e x[row of the pair]) for every pair of expert e, tile by tile, so that an
//                    expert's weights are read once per tile of its rows.  Two modes: gate and up product with the
//                    activation (x = the token's row; out [pairs, ff]), and the down product times the pair's weight
//                    (x = the pair's activated row; out [pairs, hidden]).  float32 and odd sizes run FFMA tiles whose
//                    sums over k have a fixed order; bfloat16 runs mma.sync m16n8k16 tiles fed by cp.async.
//   li_moe_combine   out[token] = sum over its slots of the pairs' rows, in slot order, in 32-bit.
//   li_moe_router    the router's 32-bit product and li_moe_route in one launch.
//   li_moe_gather    the pairs' token rows in the order of the experts' runs: the first operand of the grouped product
//                    on the fifth-generation tensor cores (gemm_tcgen05.cu), which wants an expert's rows side by side.
//
// Activations of an expert (32-bit): 0: silu(g) * u.  1: g' = min(g, limit), u' = clamp(u, -limit, limit),
// g' * sigmoid(alpha * g') * (u' + 1).
#include "attention_mma.cuh"

namespace li {

constexpr int kModeGateUp = 0, kModeDown = 1;

__device__ __forceinline__ float expert_activation(float g, float u, int act, float limit, float alpha) {
  if (act == 1) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f);
  }
  return g * (1.0f / (1.0f + expf(-g))) * u;
}

// ------------------------------------------------------------------------------------------ route
// The index of the largest of v[0..n) (ties: the lowest index); every lane gets it.  Entries are scores >= 0 or marks
// of -1 and -2; whatever they hold, the result is an index below n (a row of padding may bring anything).
__device__ __forceinline__ int warp_argmax(const float* v, int n, int lane) {
  float best = -3.0f;
  int at = 0x7fffffff;
  for (int i = lane; i < n; i += 32)
    if (v[i] > best) { best = v[i]; at = i; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa = __shfl_xor_sync(0xffffffffu, at, o);
    if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
  }
  return min(at, n - 1);
}

constexpr int kRouteWarps = 4;

// One warp routes one token: z [experts] its logits; sc [experts] and gb [groups] scratch in shared memory (sc may be z).
__device__ __forceinline__ void route_token(const float* z, float* sc, float* gb, int lane, int t, int experts, int top,
                                            int groups, int keep, int renormalise, int* __restrict__ ids,
                                            float* __restrict__ weights) {
  float mx = -INFINITY;
  for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < experts; e += 32) {
    const float v = expf(z[e] - mx);
    sc[e] = v;
    sum += v;
  }
  const float inv = 1.0f / warp_sum(sum);
  for (int e = lane; e < experts; e += 32) {
    const float score = sc[e] * inv;
    sc[e] = score >= 0.f ? score : 0.f;       // a row of padding may hold anything, NaN too: its choice stays an expert
  }
  __syncwarp();
  if (groups > 1) {
    const int per = experts / groups;
    for (int g = lane; g < groups; g += 32) {
      float best = 0.f;
      for (int j = 0; j < per; ++j) best = fmaxf(best, sc[g * per + j]);
      gb[g] = best;
    }
    __syncwarp();
    for (int r = 0; r < keep; ++r) {          // a kept group is marked by -2 (scores are never negative)
      const int g = warp_argmax(gb, groups, lane);
      __syncwarp();
      if (lane == 0) gb[g] = -2.0f;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (gb[e / per] != -2.0f) sc[e] = -1.0f;
    __syncwarp();
  }
  float total = 0.f;
  for (int r = 0; r < top; ++r) {
    const int e = warp_argmax(sc, experts, lane);
    const float w = sc[e];
    total += w;
    __syncwarp();
    if (lane == 0) {
      ids[(size_t)t * top + r] = e;
      weights[(size_t)t * top + r] = w;
      sc[e] = -1.0f;
    }
    __syncwarp();
  }
  if (renormalise && lane < top) weights[(size_t)t * top + lane] /= total;     // (top <= 32 where this is asked for)
}

__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_kernel(const float* __restrict__ logits, int tokens, int experts, int top, int groups, int keep,
                 int renormalise, int* __restrict__ ids, float* __restrict__ weights) {
  extern __shared__ float route_smem[];       // per warp: scores[experts], group scores[groups]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  grid_dependency_wait();
  if (t >= tokens) return;
  float* sc = route_smem + warp * (experts + groups);
  route_token(logits + (size_t)t * experts, sc, sc + experts, lane, t, experts, top, groups, keep, renormalise, ids,
              weights);
}

// The router's product and the routing in one launch: logits[e] = sum_k x[k] * w[e][k] in 32-bit (lane l adds up
// k = l, l + 32, ..., then the lanes' sums meet in a fixed tree: the same bits whatever else is in the step), then
// `route_token`.  A block takes TOK tokens; its warps take the experts in turn: eight warps for eight tokens of a wide
// step, thirty-two for the one token of a narrow step, where a warp's chain of loads is what the launch waits for.
template <typename T, int TOK, int kRouterWarps>
__global__ void __launch_bounds__(kRouterWarps * 32)
moe_router_kernel(const T* __restrict__ x, size_t x_stride, const float* __restrict__ w, int tokens, int K, int experts,
                  int top, int groups, int keep, int renormalise, int* __restrict__ ids, float* __restrict__ weights) {
  extern __shared__ float route_smem[];       // TOK x (logits[experts], group scores[groups])
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * TOK;
  grid_dependency_wait();
  // Four k a lane and round where the rows allow 16-byte reads (several rounds' loads are in flight at once), else one.
  const bool wide = (K % 4) == 0 && (x_stride % 4) == 0 && aligned16(w) && (reinterpret_cast<uintptr_t>(x) % (4 * sizeof(T))) == 0;
  for (int e = warp; e < experts; e += kRouterWarps) {
    const float* we = w + (size_t)e * K;
    float acc[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) acc[t] = 0.f;
    if (wide) {
#pragma unroll 8
      for (int k = lane * 4; k < K; k += 128) {
        const float4 wv = *reinterpret_cast<const float4*>(we + k);
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
          if (t0 + t >= tokens) continue;
          const T* xr = x + (size_t)(t0 + t) * x_stride + k;
          float x0, x1, x2, x3;
          if (sizeof(T) == 4) {
            const float4 xv = *reinterpret_cast<const float4*>(xr);
            x0 = xv.x; x1 = xv.y; x2 = xv.z; x3 = xv.w;
          } else {
            const uint2 xv = *reinterpret_cast<const uint2*>(xr);
            x0 = __uint_as_float(xv.x << 16); x1 = __uint_as_float(xv.x & 0xffff0000u);
            x2 = __uint_as_float(xv.y << 16); x3 = __uint_as_float(xv.y & 0xffff0000u);
          }
          acc[t] = fmaf(x3, wv.w, fmaf(x2, wv.z, fmaf(x1, wv.y, fmaf(x0, wv.x, acc[t]))));
        }
      }
    } else {
      for (int k = lane; k < K; k += 32) {
        const float wv = we[k];
#pragma unroll
        for (int t = 0; t < TOK; ++t)
          if (t0 + t < tokens) acc[t] = fmaf(to_float(x[(size_t)(t0 + t) * x_stride + k]), wv, acc[t]);
      }
    }
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      const float sum = warp_sum(acc[t]);
      if (lane == 0) route_smem[t * (experts + groups) + e] = sum;
    }
  }
  __syncthreads();
  if (warp < TOK && t0 + warp < tokens) {
    float* sc = route_smem + warp * (experts + groups);
    route_token(sc, sc, sc + experts, lane, t0 + warp, experts, top, groups, keep, renormalise, ids, weights);
  }
}

// ------------------------------------------------------------------------------------------- sort
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int pairs, int experts, int tile_rows, int* __restrict__ offsets,
                int* __restrict__ order, int* __restrict__ tile_expert, int* __restrict__ tile_row0, int max_tiles,
                int* __restrict__ place) {
  extern __shared__ int sort_smem[];          // counts[experts], cursor[experts]
  int* counts = sort_smem;
  int* cursor = sort_smem + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  grid_dependency_wait();
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < experts) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, tile = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = run;
      cursor[e] = run;
      const int n = counts[e];
      for (int r = 0; r < n && tile < max_tiles; r += tile_rows, ++tile) {
        tile_expert[tile] = e;
        tile_row0[tile] = run + r;
      }
      run += n;
    }
    offsets[experts] = run;
    for (; tile < max_tiles; ++tile) tile_expert[tile] = -1;
  }
  __syncthreads();
  // The order of an expert's rows among themselves does not matter: every row of the products is computed alone.
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < experts) {
      const int at = atomicAdd(&cursor[e], 1);
      order[at] = i;
      if (place != nullptr) place[i] = at;
    }
  }
}

// out[m] = x[order[m] / top]: every pair's token row, in the order of the experts' runs.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, size_t x_stride, const int* __restrict__ order, int top,
                                  T* __restrict__ out, int pairs, int width) {
  constexpr int N = Vec16<T>::N;
  grid_dependency_wait();
  const int per_row = width / N;
  const size_t total = (size_t)pairs * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / per_row), c = (int)(i - (size_t)m * per_row) * N;
    store16(out + (size_t)m * width + c, load16(x + (size_t)(order[m] / top) * x_stride + c));
  }
}

// --------------------------------------------------------------------------------- grouped, FFMA
constexpr int kSimtRows = 32;       // rows of a tile

// The row of an expert's [2N, K] matrix that holds column `col` of the gate (or of the up) product: the gate rows,
// then the up rows; or, `eights`, both interleaved in eights (eight gate rows, then their eight up rows).
__device__ __forceinline__ int gate_up_row(int col, bool up, int N, int eights) {
  return eights ? (col >> 3) * 16 + (up ? 8 : 0) + (col & 7) : (up ? N : 0) + col;
}

// a: rows of `a_stride`; w: [experts][rows of W][K] with rows of W = 2N (gate rows, then up rows) or N (down).
// A block: one tile of rows of one expert x 64 rows of W (gate/up: 32 of each for the same 32 columns).
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_grouped_simt_kernel(const T* __restrict__ a, size_t a_stride, const T* __restrict__ w, T* __restrict__ out,
                        size_t out_stride, const int* __restrict__ order, const int* __restrict__ offsets,
                        const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                        const float* __restrict__ pair_weights, int top, int N, int K, int act, float limit,
                        float alpha, int eights) {
  __shared__ float As[kSimtRows][33];
  __shared__ float Bs[64][33];
  __shared__ int src_rows[kSimtRows], out_rows[kSimtRows];
  grid_dependency_wait();
  const int e = tile_expert[blockIdx.x];
  if (e < 0) return;
  const int row0 = tile_row0[blockIdx.x];
  const int rows = min(kSimtRows, offsets[e + 1] - row0);
  if (threadIdx.x < kSimtRows) {
    const int pair = threadIdx.x < rows ? order[row0 + threadIdx.x] : -1;
    out_rows[threadIdx.x] = pair;
    src_rows[threadIdx.x] = pair < 0 ? -1 : (MODE == kModeGateUp ? pair / top : pair);
  }
  __syncthreads();
  const int n0 = blockIdx.y * (MODE == kModeGateUp ? 32 : 64);
  const T* we = w + (size_t)e * (MODE == kModeGateUp ? 2 * N : N) * K;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  for (int k0 = 0; k0 < K; k0 += 32) {
    for (int i = threadIdx.x; i < kSimtRows * 32; i += 256) {
      const int r = i >> 5, c = i & 31;
      const int src = src_rows[r];
      As[r][c] = (src >= 0 && k0 + c < K) ? to_float(a[(size_t)src * a_stride + k0 + c]) : 0.f;
    }
    for (int i = threadIdx.x; i < 64 * 32; i += 256) {
      const int r = i >> 5, c = i & 31;
      int wrow;
      bool ok;
      if (MODE == kModeGateUp) { ok = n0 + (r & 31) < N; wrow = gate_up_row(n0 + (r & 31), r >= 32, N, eights); }
      else { ok = n0 + r < N; wrow = n0 + r; }
      Bs[r][c] = (ok && k0 + c < K) ? to_float(we[(size_t)wrow * K + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < 32; ++kk) {
      const float a0 = As[ty * 2][kk], a1 = As[ty * 2 + 1][kk];
      const float b0 = Bs[2 * tx][kk], b1 = Bs[2 * tx + 1][kk], b2 = Bs[32 + 2 * tx][kk], b3 = Bs[33 + 2 * tx][kk];
      acc[0][0] = fmaf(a0, b0, acc[0][0]); acc[0][1] = fmaf(a0, b1, acc[0][1]);
      acc[0][2] = fmaf(a0, b2, acc[0][2]); acc[0][3] = fmaf(a0, b3, acc[0][3]);
      acc[1][0] = fmaf(a1, b0, acc[1][0]); acc[1][1] = fmaf(a1, b1, acc[1][1]);
      acc[1][2] = fmaf(a1, b2, acc[1][2]); acc[1][3] = fmaf(a1, b3, acc[1][3]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int pair = out_rows[ty * 2 + i];
    if (pair < 0) continue;
    T* orow = out + (size_t)pair * out_stride;
    if (MODE == kModeGateUp) {
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (n0 + 2 * tx + j < N)
          orow[n0 + 2 * tx + j] = from_float<T>(expert_activation(acc[i][j], acc[i][2 + j], act, limit, alpha));
    } else {
      const float scale = pair_weights != nullptr ? pair_weights[pair] : 1.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = n0 + (j < 2 ? 0 : 32) + 2 * tx + (j & 1);
        if (col < N) orow[col] = from_float<T>(acc[i][j] * scale);
      }
    }
  }
}

// ----------------------------------------------------------------------------- grouped, mma.sync
constexpr int kMmaRows = 64;        // rows of a tile
constexpr int kMmaK = 64, kMmaLd = kMmaK + 8;

template <int MODE>
__global__ void __launch_bounds__(128)
moe_grouped_mma_kernel(const bf16* __restrict__ a, size_t a_stride, const bf16* __restrict__ w, bf16* __restrict__ out,
                       size_t out_stride, const int* __restrict__ order, const int* __restrict__ offsets,
                       const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                       const float* __restrict__ pair_weights, int top, int N, int K, int act, float limit,
                       float alpha, int eights) {
  __shared__ __align__(16) bf16 As[2][kMmaRows * kMmaLd];
  __shared__ __align__(16) bf16 Bs[2][64 * kMmaLd];
  __shared__ int src_rows[kMmaRows], out_rows[kMmaRows];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  grid_dependency_wait();
  const int e = tile_expert[blockIdx.x];
  if (e < 0) return;
  const int row0 = tile_row0[blockIdx.x];
  const int rows = min(kMmaRows, offsets[e + 1] - row0);
  if (tid < kMmaRows) {
    const int pair = tid < rows ? order[row0 + tid] : -1;
    out_rows[tid] = pair;
    src_rows[tid] = pair < 0 ? -1 : (MODE == kModeGateUp ? pair / top : pair);
  }
  __syncthreads();
  const int n0 = blockIdx.y * (MODE == kModeGateUp ? 32 : 64);
  const bf16* we = w + (size_t)e * (MODE == kModeGateUp ? 2 * N : N) * K;

  auto load = [&](int buf, int k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 128, r = idx >> 3, c = idx & 7, k = k0 + c * 8;
      const int src = src_rows[r];
      const bool valid = src >= 0 && k < K;
      cp_async16(&As[buf][r * kMmaLd + c * 8], valid ? a + (size_t)src * a_stride + k : a, valid);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 128, r = idx >> 3, c = idx & 7, k = k0 + c * 8;
      int wrow;
      bool ok;
      if (MODE == kModeGateUp) { ok = n0 + (r & 31) < N; wrow = gate_up_row(n0 + (r & 31), r >= 32, N, eights); }
      else { ok = n0 + r < N; wrow = n0 + r; }
      const bool valid = ok && k < K;
      cp_async16(&Bs[buf][r * kMmaLd + c * 8], valid ? we + (size_t)wrow * K + k : we, valid);
    }
    cp_async_commit();
  };

  float acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const int nk = (K + kMmaK - 1) / kMmaK;
  load(0, 0);
  for (int kt = 0; kt < nk; ++kt) {
    if (kt + 1 < nk) {
      load((kt + 1) & 1, (kt + 1) * kMmaK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* as = As[kt & 1];
    const bf16* bs = Bs[kt & 1];
#pragma unroll
    for (int kk = 0; kk < kMmaK / 16; ++kk) {
      unsigned af[4];
      ldmatrix_x4(af[0], af[1], af[2], af[3], as + (warp * 16 + (lane & 15)) * kMmaLd + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nn = 0; nn < 4; ++nn) {
        unsigned b0, b1, b2, b3;
        const int mtx = lane >> 3;
        ldmatrix_x4(b0, b1, b2, b3, bs + (nn * 16 + (mtx >> 1) * 8 + (lane & 7)) * kMmaLd + kk * 16 + (mtx & 1) * 8);
        mma_bf16(acc[nn * 2], af, b0, b1);
        mma_bf16(acc[nn * 2 + 1], af, b2, b3);
      }
    }
    __syncthreads();      // this buffer is overwritten by the load issued in the next iteration
  }

  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int pair = out_rows[warp * 16 + g + 8 * h];
    if (pair < 0) continue;
    bf16* orow = out + (size_t)pair * out_stride;
    if (MODE == kModeGateUp) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = n0 + j * 8 + 2 * t;
        if (col < N)
          *reinterpret_cast<unsigned*>(orow + col) =
              pack_bf16(expert_activation(acc[j][2 * h], acc[j + 4][2 * h], act, limit, alpha),
                        expert_activation(acc[j][2 * h + 1], acc[j + 4][2 * h + 1], act, limit, alpha));
      }
    } else {
      const float scale = pair_weights != nullptr ? pair_weights[pair] : 1.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = n0 + j * 8 + 2 * t;
        if (col < N) *reinterpret_cast<unsigned*>(orow + col) = pack_bf16(acc[j][2 * h] * scale, acc[j][2 * h + 1] * scale);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------- combine
// `kVec`: 16 bytes of a row a thread (width a multiple of the vector's length); the sums are the same either way.
template <typename T, bool kVec>
__global__ void moe_combine_kernel(const T* __restrict__ y, T* __restrict__ out, size_t tokens, int top, int width,
                                   const int* __restrict__ place) {
  constexpr int N = kVec ? Vec16<T>::N : 1;
  grid_dependency_wait();
  const size_t per_row = (size_t)width / N, total = tokens * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / per_row, c = (i - t * per_row) * N;
    float sum[N];
#pragma unroll
    for (int e = 0; e < N; ++e) sum[e] = 0.f;
    for (int s = 0; s < top; ++s) {
      const size_t row = place != nullptr ? (size_t)place[t * top + s] : t * top + s;
      if (kVec) {
        float v[Vec16<T>::N];
        unpack16(load16(y + row * width + c), v);
#pragma unroll
        for (int e = 0; e < N; ++e) sum[e] += v[e];
      } else {
        sum[0] += to_float(y[row * width + c]);
      }
    }
    if (kVec) {
      Vec16<T> o;
#pragma unroll
      for (int e = 0; e < N; ++e) o.set(e, sum[e]);
      store16(out + t * width + c, o);
    } else {
      out[t * width + c] = from_float<T>(sum[0]);
    }
  }
}

template <typename T, int MODE>
static int launch_simt(const void* a, size_t a_stride, const void* w, void* out, size_t out_stride, const int* order,
                       const int* offsets, const int* tile_expert, const int* tile_row0, const float* pair_weights,
                       int top, int N, int K, int act, float limit, float alpha, int max_tiles, int eights,
                       cudaStream_t stream) {
  const dim3 grid(max_tiles, MODE == kModeGateUp ? (N + 31) / 32 : (N + 63) / 64);
  return (int)launch_pdl(max_tiles, moe_grouped_simt_kernel<T, MODE>, grid, dim3(256), 0, stream, (const T*)a, a_stride,
                         (const T*)w, (T*)out, out_stride, order, offsets, tile_expert, tile_row0, pair_weights, top, N,
                         K, act, limit, alpha, eights);
}

template <int MODE>
static int launch_mma(const void* a, size_t a_stride, const void* w, void* out, size_t out_stride, const int* order,
                      const int* offsets, const int* tile_expert, const int* tile_row0, const float* pair_weights,
                      int top, int N, int K, int act, float limit, float alpha, int max_tiles, int eights,
                      cudaStream_t stream) {
  const dim3 grid(max_tiles, MODE == kModeGateUp ? (N + 31) / 32 : (N + 63) / 64);
  return (int)launch_pdl(max_tiles, moe_grouped_mma_kernel<MODE>, grid, dim3(128), 0, stream, (const bf16*)a, a_stride,
                         (const bf16*)w, (bf16*)out, out_stride, order, offsets, tile_expert, tile_row0, pair_weights,
                         top, N, K, act, limit, alpha, eights);
}

}  // namespace li

using namespace li;

// logits [tokens, experts] float; ids [tokens, top] int; weights [tokens, top] float.
LI_EXPORT int li_moe_route(const float* logits, int tokens, int experts, int top, int groups, int keep,
                           int renormalise, int* ids, float* weights, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (experts < 1 || top < 1 || top > experts || groups < 1 || experts % groups || keep < 1 || keep > groups)
    return LI_ERR_UNSUPPORTED;
  if (keep * (experts / groups) < top || (renormalise && top > 32)) return LI_ERR_UNSUPPORTED;
  const size_t smem = (size_t)kRouteWarps * (experts + groups) * sizeof(float);
  if (smem > 48 * 1024) return LI_ERR_UNSUPPORTED;
  return (int)launch_pdl(tokens, moe_route_kernel, dim3((tokens + kRouteWarps - 1) / kRouteWarps), dim3(kRouteWarps * 32),
                         smem, stream, logits, tokens, experts, top, groups, keep, renormalise, ids, weights);
}

// Rows of a tile of the grouped product that li_moe_grouped will run for this dtype and these sizes.
LI_EXPORT int li_moe_tile_rows(int dtype, int N, int K) {
  return (dtype == kBFloat16 && K % 8 == 0 && N % 2 == 0) ? kMmaRows : kSimtRows;
}

// ids [pairs] int (the expert of every pair); offsets [experts + 1]; order [pairs]; tile_expert, tile_row0 [max_tiles]
// with max_tiles >= pairs / tile_rows + experts.
// place [pairs] (optional): where in `order` each pair stands.
LI_EXPORT int li_moe_sort(const int* ids, int pairs, int experts, int tile_rows, int* offsets, int* order,
                          int* tile_expert, int* tile_row0, int max_tiles, int* place, cudaStream_t stream) {
  if (experts < 1 || tile_rows < 1 || max_tiles < (pairs + tile_rows - 1) / tile_rows + experts - 1)
    return LI_ERR_UNSUPPORTED;
  const size_t smem = (size_t)2 * experts * sizeof(int);
  if (smem > 48 * 1024) return LI_ERR_UNSUPPORTED;
  return (int)launch_pdl(pairs, moe_sort_kernel, dim3(1), dim3(1024), smem, stream, ids, pairs, experts, tile_rows,
                         offsets, order, tile_expert, tile_row0, max_tiles, place);
}

// x [tokens, K] (rows x_stride apart) in the engine's dtype, w [experts, K] float: the router's product and the routing
// of li_moe_route in one launch.
LI_EXPORT int li_moe_router(int dtype, const void* x, size_t x_stride, const float* w, int tokens, int K, int experts,
                            int top, int groups, int keep, int renormalise, int* ids, float* weights,
                            cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (experts < 1 || top < 1 || top > experts || groups < 1 || experts % groups || keep < 1 || keep > groups || K < 1)
    return LI_ERR_UNSUPPORTED;
  if (keep * (experts / groups) < top || (renormalise && top > 32)) return LI_ERR_UNSUPPORTED;
  const bool wide = tokens > 128;
  const size_t smem = (size_t)(wide ? 8 : 1) * (experts + groups) * sizeof(float);
  if (smem > 48 * 1024) return LI_ERR_UNSUPPORTED;
#define LI_ROUTER(T, TOK, WARPS)                                                                                      \
  return (int)launch_pdl(tokens, moe_router_kernel<T, TOK, WARPS>, dim3((tokens + TOK - 1) / TOK), dim3(WARPS * 32),   \
                         smem, stream, (const T*)x, x_stride, w, tokens, K, experts, top, groups, keep, renormalise,  \
                         ids, weights)
  if (dtype == kFloat32) { if (wide) LI_ROUTER(float, 8, 8); LI_ROUTER(float, 1, 32); }
  if (wide) LI_ROUTER(bf16, 8, 8);
  LI_ROUTER(bf16, 1, 32);
#undef LI_ROUTER
}

// out [pairs, width] = x[order[m] / top] for every place m of `order`; width a multiple of 16 bytes.
LI_EXPORT int li_moe_gather(int dtype, const void* x, size_t x_stride, const int* order, int top, void* out, int pairs,
                            int width, cudaStream_t stream) {
  if (pairs == 0 || width == 0) return 0;
  const int n = dtype == kFloat32 ? 4 : 8;
  if (width % n || x_stride % n || !aligned16(x) || !aligned16(out)) return LI_ERR_ALIGNMENT;
  const size_t total = (size_t)pairs * (width / n);
  const dim3 grid((unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16));
  if (dtype == kFloat32)
    return (int)launch_pdl(pairs, moe_gather_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, x_stride, order,
                           top, (float*)out, pairs, width);
  return (int)launch_pdl(pairs, moe_gather_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)x, x_stride, order, top,
                         (bf16*)out, pairs, width);
}

// mode 0: out[pair, 0:N] = act(W_gate,e x[pair / top], W_up,e x[pair / top]), w [experts, 2N, K] (gate rows, then up).
// mode 1: out[pair, 0:N] = (W_down,e a[pair]) * pair_weights[pair] (null: 1), w [experts, N, K].
// `tile_rows`: the rows of the tiles li_moe_sort made: 64 runs the tensor-core tiles (only where
// li_moe_tile_rows(dtype, N, K) says 64), 32 the FFMA tiles.
LI_EXPORT int li_moe_grouped(int dtype, int mode, const void* a, size_t a_stride, const void* w, void* out,
                             size_t out_stride, const int* order, const int* offsets, const int* tile_expert,
                             const int* tile_row0, const float* pair_weights, int top, int N, int K, int act,
                             float limit, float alpha, int max_tiles, int tile_rows, int eights,
                             cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0 || K <= 0) return 0;
  if (tile_rows != kSimtRows && !(tile_rows == kMmaRows && li_moe_tile_rows(dtype, N, K) == kMmaRows))
    return LI_ERR_UNSUPPORTED;
  if (mode != kModeGateUp && mode != kModeDown) return LI_ERR_UNSUPPORTED;
  if (eights && mode == kModeGateUp && (N % 8)) return LI_ERR_UNSUPPORTED;
  if (max_tiles > 0x7fffffff / 2 || (N + 31) / 32 > 65535) return LI_ERR_UNSUPPORTED;
#define LI_MOE_ARGS a, a_stride, w, out, out_stride, order, offsets, tile_expert, tile_row0, pair_weights, top, N, K, act, \
                    limit, alpha, max_tiles, eights, stream
  if (dtype == kFloat32)
    return mode == kModeGateUp ? launch_simt<float, kModeGateUp>(LI_MOE_ARGS) : launch_simt<float, kModeDown>(LI_MOE_ARGS);
  if (tile_rows == kMmaRows) {
    if ((a_stride % 8) || (out_stride % 2) || !aligned16(a) || !aligned16(w) || (reinterpret_cast<uintptr_t>(out) & 3))
      return LI_ERR_ALIGNMENT;
    return mode == kModeGateUp ? launch_mma<kModeGateUp>(LI_MOE_ARGS) : launch_mma<kModeDown>(LI_MOE_ARGS);
  }
  return mode == kModeGateUp ? launch_simt<bf16, kModeGateUp>(LI_MOE_ARGS) : launch_simt<bf16, kModeDown>(LI_MOE_ARGS);
#undef LI_MOE_ARGS
}

// out [tokens, width] = sum over s < top of y[row of pair token * top + s, :], in slot order; the row is the pair
// itself, or place[pair] where `place` is given (rows in the order of the experts' runs).
LI_EXPORT int li_moe_combine(int dtype, const void* y, void* out, int tokens, int top, int width, const int* place,
                             cudaStream_t stream) {
  if ((size_t)tokens * width == 0) return 0;
  const int n = dtype == kFloat32 ? 4 : 8;
  const bool vec = width % n == 0 && aligned16(y) && aligned16(out);
  const size_t total = (size_t)tokens * width / (vec ? n : 1);
  const dim3 grid((unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16));
#define LI_COMBINE(T, V)                                                                                             \
  return (int)launch_pdl(tokens, moe_combine_kernel<T, V>, grid, dim3(256), 0, stream, (const T*)y, (T*)out,          \
                         (size_t)tokens, top, width, place)
  if (dtype == kFloat32) { if (vec) LI_COMBINE(float, true); LI_COMBINE(float, false); }
  if (vec) LI_COMBINE(bf16, true);
  LI_COMBINE(bf16, false);
#undef LI_COMBINE
}
