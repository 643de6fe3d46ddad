// Norms of a model whose residual stream is summed in 32-bit, and the casts around that stream.
//
//   li_convert             dst = src between float and bfloat16 (rows may be column slices of wider tensors)
//   li_layernorm           v = x[row] (+ w_d * norm(value[row]));  x[row] = v (optional);  out = w * norm(v)
//                          norm(v) = (v - mean) / sqrt(var + eps), var = mean of squared deviations; one block a row.
//                          Either norm may be a root-mean-square norm instead (no mean taken off), out may be the
//                          sum v itself (rounded to the engine's type: what a sublayer reads of a 32-bit stream
//                          that is normalised only on its way back), and the weights may be 32-bit
//   li_projection_rmsnorm  x = w * x / sqrt(mean(x^2) + eps) in place over whole rows of one or two neighbouring
//                          column slices (q and k of a fused projection, each normalised across all its heads)
//   li_gated_rmsnorm       out = w * x / sqrt(mean(x^2) + eps) * act(gate) per head; one warp a (token, head);
//                          act = silu or sigmoid; w shared by the heads or one per head; x optionally divided by
//                          a number per (token, head) first
//
// x of li_layernorm may be float while value, weights and out are bfloat16: the stream stays 32-bit, what the
// products read is rounded once.  Means, variances, the sum into the stream and every product before the final
// rounding are 32-bit; the variance is taken in a second pass over the centred row, which the block keeps in
// shared memory.  The order of every sum depends on the row's width only.
#include "common.cuh"

namespace li {

template <typename S, typename D>
__global__ void convert_kernel(const S* __restrict__ src, size_t src_stride, D* __restrict__ dst, size_t dst_stride,
                               int rows, int width) {
  grid_dependency_wait();
  const size_t total = (size_t)rows * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / width, c = i - r * width;
    dst[r * dst_stride + c] = from_float<D>(to_float(src[r * src_stride + c]));
  }
}

// Mean and 1 / sqrt(var + eps) of the `width` floats in `row` (shared memory); with `centre` false the mean is 0.
__device__ __forceinline__ void row_statistics(const float* row, int width, float eps, bool centre, float* scratch,
                                               float& mean, float& inv) {
  mean = 0.f;
  if (centre) {
    float s = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) s += row[c];
    mean = block_sum(s, scratch) / (float)width;
  }
  float q = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float d = row[c] - mean;
    q += d * d;
  }
  const float var = block_sum(q, scratch) / (float)width;
  inv = 1.0f / sqrtf(var + eps);
}

// T: dtype of value and out.  X: dtype of the stream x.  W: dtype of the weights.  value_centre / centre: whether
// the delta's norm / the norm of the sum takes the mean off; plain_out: out is the sum itself.
template <typename T, typename X, typename W>
__global__ void __launch_bounds__(1024)
layernorm_kernel(X* __restrict__ x, const T* __restrict__ value, const W* __restrict__ value_weight,
                 const W* __restrict__ weight, T* __restrict__ out, const int* __restrict__ rows, int width, float eps,
                 float value_eps, int write_stream, int centre, int value_centre, int plain_out) {
  extern __shared__ float row[];  // [width]
  __shared__ float scratch[33];
  grid_dependency_wait();
  const int r = blockIdx.x;
  const size_t at = (size_t)(rows ? rows[r] : r) * width;
  float mean, inv;
  if (value != nullptr) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = to_float(value[at + c]);
    __syncthreads();
    row_statistics(row, width, value_eps, value_centre != 0, scratch, mean, inv);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      const float normed = (row[c] - mean) * inv * to_float(value_weight[c]);
      const float v = to_float(x[at + c]) + normed;
      if (write_stream) x[at + c] = from_float<X>(v);
      row[c] = round_to<X>(v);
    }
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = to_float(x[at + c]);
  }
  if (out == nullptr) return;
  __syncthreads();
  T* o = out + (size_t)r * width;
  if (plain_out) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = from_float<T>(row[c]);
    return;
  }
  row_statistics(row, width, eps, centre != 0, scratch, mean, inv);
  for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = from_float<T>((row[c] - mean) * inv * to_float(weight[c]));
}

// Four neighbouring elements as floats, by one 16-byte (float) or 8-byte (bfloat16) access.
__device__ __forceinline__ void load4(const float* p, float (&o)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&o)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);      // widened with shifts and masks (see unpack16)
  o[0] = __uint_as_float(raw.x << 16); o[1] = __uint_as_float(raw.x & 0xffff0000u);
  o[2] = __uint_as_float(raw.y << 16); o[3] = __uint_as_float(raw.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<const unsigned*>(&a);
  raw.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// The same norm with the row in registers: thread i keeps the four-element chunks i, i + blockDim, ... (NV of them).
// For widths that are multiples of four and at most 4 * NV * blockDim, and 16-byte aligned rows.
template <typename T, typename X, typename W, int NV>
__global__ void __launch_bounds__(1024)
layernorm_rows_kernel(X* __restrict__ x, const T* __restrict__ value, const W* __restrict__ value_weight,
                      const W* __restrict__ weight, T* __restrict__ out, const int* __restrict__ rows, int width,
                      float eps, float value_eps, int write_stream, int centre, int value_centre, int plain_out) {
  __shared__ float scratch[33];
  // The weights are inputs of the model, not of a kernel: they are on their way before the wait.
  float w[NV][4], wd[NV][4];
  int col[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    col[i] = (i * blockDim.x + threadIdx.x) * 4;
    if (col[i] < width) {
      if (weight != nullptr && !plain_out) load4(weight + col[i], w[i]);
      if (value != nullptr) load4(value_weight + col[i], wd[i]);
    }
  }
  grid_dependency_wait();
  const int r = blockIdx.x;
  const size_t at = (size_t)(rows ? rows[r] : r) * width;
  const float n = (float)width;
  float v[NV][4];
  if (value != nullptr) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (col[i] < width) {
        load4(value + at + col[i], v[i]);
        s += (v[i][0] + v[i][1]) + (v[i][2] + v[i][3]);
      }
    }
    const float mean = value_centre ? block_sum(s, scratch) / n : 0.f;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (col[i] < width)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[i][e] -= mean;
          q = fmaf(v[i][e], v[i][e], q);
        }
    const float inv = 1.0f / sqrtf(block_sum(q, scratch) / n + value_eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (col[i] < width) {
        float base[4];
        load4(x + at + col[i], base);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[i][e] = base[e] + v[i][e] * inv * wd[i][e];
        if (write_stream) store4(x + at + col[i], v[i]);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[i][e] = round_to<X>(v[i][e]);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (col[i] < width) load4(x + at + col[i], v[i]);
  }
  if (out == nullptr) return;
  if (plain_out) {
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (col[i] < width) store4(out + (size_t)r * width + col[i], v[i]);
    return;
  }
  float mean = 0.f;
  if (centre) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (col[i] < width) s += (v[i][0] + v[i][1]) + (v[i][2] + v[i][3]);
    mean = block_sum(s, scratch) / n;
  }
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i)
    if (col[i] < width)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[i][e] -= mean;
        q = fmaf(v[i][e], v[i][e], q);
      }
  const float inv = 1.0f / sqrtf(block_sum(q, scratch) / n + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (col[i] < width) {
#pragma unroll
      for (int e = 0; e < 4; ++e) v[i][e] = v[i][e] * inv * w[i][e];
      store4(out + (size_t)r * width + col[i], v[i]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
projection_rmsnorm_kernel(T* __restrict__ x, size_t stride, int width_a, const T* __restrict__ weight_a, int width_b,
                          const T* __restrict__ weight_b, float eps) {
  __shared__ float scratch[33];
  grid_dependency_wait();
  const bool second = blockIdx.y == 1;
  T* p = x + (size_t)blockIdx.x * stride + (second ? width_a : 0);
  const int width = second ? width_b : width_a;
  const T* w = second ? weight_b : weight_a;
  float q = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_float(p[c]);
    q += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) p[c] = from_float<T>(to_float(p[c]) * inv * to_float(w[c]));
}

// weight_stride: 0 = one weight vector for every head, `size` = one per head.  act: 0 silu, 1 sigmoid.  den (may
// be null): x[t, h] is divided by den[t * heads + h] before anything else.
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ x, const T* __restrict__ gate, size_t gate_stride,
                                     const float* __restrict__ weight, T* __restrict__ out, int tokens, int heads,
                                     int size, float eps, int weight_stride, int act, const float* __restrict__ den) {
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // (token, head)
  if (item >= (size_t)tokens * heads) return;
  const size_t t = item / heads;
  const int h = (int)(item - t * heads);
  const float* xr = x + (t * heads + h) * size;
  const float under = den != nullptr ? den[item] : 1.0f;
  float q = 0.f;
  for (int c = lane; c < size; c += 32) {
    const float v = den != nullptr ? xr[c] / under : xr[c];
    q += v * v;
  }
  const float inv = 1.0f / sqrtf(warp_sum(q) / (float)size + eps);
  const T* g = gate + t * gate_stride + (size_t)h * size;
  const float* w = weight + (size_t)h * weight_stride;
  T* o = out + (t * heads + h) * size;
  for (int c = lane; c < size; c += 32) {
    const float z = to_float(g[c]);
    const float s = 1.0f / (1.0f + expf(-z));
    const float v = den != nullptr ? xr[c] / under : xr[c];
    o[c] = from_float<T>(v * inv * w[c] * (act == 1 ? s : z * s));
  }
}

// The same with 16-byte accesses: a lane keeps NV groups of four of its head's row in registers between the sum
// of squares and the scaling.  size a multiple of four and at most 128 NV; every row 16-byte (gate: 8-byte in
// bfloat16) aligned.
template <typename T, int NV>
__global__ void gated_rmsnorm_vec_kernel(const float* __restrict__ x, const T* __restrict__ gate, size_t gate_stride,
                                         const float* __restrict__ weight, T* __restrict__ out, int tokens, int heads,
                                         int size, float eps, int weight_stride, int act,
                                         const float* __restrict__ den) {
  const int lane = threadIdx.x & 31;
  const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // (token, head)
  if (item >= (size_t)tokens * heads) return;
  const size_t t = item / heads;
  const int h = (int)(item - t * heads);
  const int quads = size >> 2;
  const float* w = weight + (size_t)h * weight_stride;
  float4 wv[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j)
    if (lane + 32 * j < quads) wv[j] = *reinterpret_cast<const float4*>(w + 4 * (lane + 32 * j));
  grid_dependency_wait();
  const float* xr = x + (t * heads + h) * size;
  const T* g = gate + t * gate_stride + (size_t)h * size;
  float4 v[NV];
  float z[NV][4];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (lane + 32 * j < quads) {
      v[j] = *reinterpret_cast<const float4*>(xr + 4 * (lane + 32 * j));
      load4(g + 4 * (lane + 32 * j), z[j]);
    }
  }
  if (den != nullptr) {
    const float under = den[item];
#pragma unroll
    for (int j = 0; j < NV; ++j) { v[j].x /= under; v[j].y /= under; v[j].z /= under; v[j].w /= under; }
  }
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) q += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  const float inv = 1.0f / sqrtf(warp_sum(q) / (float)size + eps);
  T* o = out + (t * heads + h) * size;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    if (lane + 32 * j >= quads) continue;
    const float xs[4] = {v[j].x, v[j].y, v[j].z, v[j].w}, ws[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
    float r[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float s = 1.0f / (1.0f + expf(-z[j][e]));
      r[e] = xs[e] * inv * ws[e] * (act == 1 ? s : z[j][e] * s);
    }
    store4(o + 4 * (lane + 32 * j), r);
  }
}

template <typename S>
int convert_from(int dst_dtype, const void* src, size_t ss, void* dst, size_t ds, int rows, int width, dim3 grid,
                 cudaStream_t stream) {
  if (dst_dtype == kFloat32)
    return (int)launch_pdl(rows, convert_kernel<S, float>, grid, dim3(256), 0, stream, (const S*)src, ss, (float*)dst,
                           ds, rows, width);
  return (int)launch_pdl(rows, convert_kernel<S, bf16>, grid, dim3(256), 0, stream, (const S*)src, ss, (bf16*)dst, ds,
                         rows, width);
}

}  // namespace li

using namespace li;

LI_EXPORT int li_convert(int src_dtype, const void* src, size_t src_stride, int dst_dtype, void* dst, size_t dst_stride,
                         int rows, int width, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  const size_t total = (size_t)rows * width;
  const dim3 grid((unsigned)((total + 1023) / 1024 < 4096 ? (total + 1023) / 1024 : 4096));
  if (src_dtype == kFloat32) return convert_from<float>(dst_dtype, src, src_stride, dst, dst_stride, rows, width, grid, stream);
  return convert_from<bf16>(dst_dtype, src, src_stride, dst, dst_stride, rows, width, grid, stream);
}

// dtype: of value and out.  x_dtype: of the stream x.  w_dtype: of value_weight and weight (dtype, or float32).
// flags: 1 = store the sum back into x, 2 = the norm of the sum is not centred (a root-mean-square norm), 4 = the
// delta's norm is not centred, 8 = out is the sum itself, not its norm.  value == null: no delta.  out == null:
// only the sum is made.
LI_EXPORT int li_layernorm(int dtype, void* x, int x_dtype, const void* value, const void* value_weight,
                           const void* weight, void* out, const int* rows, int n, int width, float eps,
                           float value_eps, int flags, int w_dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width < 1 || (size_t)width * sizeof(float) > 200 * 1024) return LI_ERR_UNSUPPORTED;
  if (dtype == kFloat32 && (x_dtype != kFloat32 || w_dtype != kFloat32)) return LI_ERR_UNSUPPORTED;
  if (w_dtype != dtype && (w_dtype != kFloat32 || x_dtype != kFloat32)) return LI_ERR_UNSUPPORTED;
  const size_t smem = (size_t)width * sizeof(float);
  const int threads = width >= 4096 ? 1024 : width >= 1024 ? 512 : 256;
  const int write_stream = flags & 1, centre = (flags & 2) ? 0 : 1, value_centre = (flags & 4) ? 0 : 1;
  const int plain_out = (flags & 8) ? 1 : 0;
  // Rows of up to 16,384 elements that 16-byte accesses can walk stay in registers.
  const bool in_registers = width % 4 == 0 && width <= 16384 && aligned16(x) && aligned16(value) && aligned16(out) &&
                            aligned16(weight) && aligned16(value_weight);
  if (in_registers) {
    const int quads = width / 4;
    const int block = quads >= 1024 ? 1024 : ((quads + 31) / 32) * 32;
    const int per_thread = (quads + block - 1) / block;
#define LI_LAUNCH_ROWS(T, X, W, NV)                                                                                   \
  return (int)launch_pdl(n, layernorm_rows_kernel<T, X, W, NV>, dim3(n), dim3(block), 0, stream, (X*)x,               \
                         (const T*)value, (const W*)value_weight, (const W*)weight, (T*)out, rows, width, eps,        \
                         value_eps, write_stream, centre, value_centre, plain_out)
#define LI_LAUNCH_ROWS_NV(T, X, W)                                                                                    \
  {                                                                                                                   \
    if (per_thread == 1) LI_LAUNCH_ROWS(T, X, W, 1);                                                                  \
    if (per_thread == 2) LI_LAUNCH_ROWS(T, X, W, 2);                                                                  \
    LI_LAUNCH_ROWS(T, X, W, 4);                                                                                       \
  }
    if (dtype == kFloat32) LI_LAUNCH_ROWS_NV(float, float, float)
    if (w_dtype == kFloat32) LI_LAUNCH_ROWS_NV(bf16, float, float)
    if (x_dtype == kFloat32) LI_LAUNCH_ROWS_NV(bf16, float, bf16)
    LI_LAUNCH_ROWS_NV(bf16, bf16, bf16)
#undef LI_LAUNCH_ROWS_NV
#undef LI_LAUNCH_ROWS
  }
#define LI_LAUNCH_NORM(T, X, W)                                                                                       \
  {                                                                                                                   \
    if (smem > 48 * 1024) {                                                                                           \
      cudaError_t e = cudaFuncSetAttribute(layernorm_kernel<T, X, W>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                           (int)smem);                                                                \
      if (e != cudaSuccess) return (int)e;                                                                            \
    }                                                                                                                 \
    return (int)launch_pdl(n, layernorm_kernel<T, X, W>, dim3(n), dim3(threads), smem, stream, (X*)x,                 \
                           (const T*)value, (const W*)value_weight, (const W*)weight, (T*)out, rows, width, eps,      \
                           value_eps, write_stream, centre, value_centre, plain_out);                                 \
  }
  if (dtype == kFloat32) LI_LAUNCH_NORM(float, float, float)
  if (w_dtype == kFloat32) LI_LAUNCH_NORM(bf16, float, float)
  if (x_dtype == kFloat32) LI_LAUNCH_NORM(bf16, float, bf16)
  LI_LAUNCH_NORM(bf16, bf16, bf16)
#undef LI_LAUNCH_NORM
}

LI_EXPORT int li_projection_rmsnorm(int dtype, void* x, size_t stride, int rows, int width_a, const void* weight_a,
                                    int width_b, const void* weight_b, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (width_a < 1 || width_b < 0) return LI_ERR_UNSUPPORTED;
  const dim3 grid(rows, width_b > 0 ? 2 : 1);
  const int widest = width_a > width_b ? width_a : width_b;
  const int threads = widest >= 4096 ? 1024 : widest >= 1024 ? 512 : 256;
  if (dtype == kFloat32)
    return (int)launch_pdl(rows, projection_rmsnorm_kernel<float>, grid, dim3(threads), 0, stream, (float*)x, stride,
                           width_a, (const float*)weight_a, width_b, (const float*)weight_b, eps);
  return (int)launch_pdl(rows, projection_rmsnorm_kernel<bf16>, grid, dim3(threads), 0, stream, (bf16*)x, stride, width_a,
                         (const bf16*)weight_a, width_b, (const bf16*)weight_b, eps);
}

LI_EXPORT int li_gated_rmsnorm(int dtype, const float* x, const void* gate, size_t gate_stride, const float* weight,
                               void* out, int tokens, int heads, int size, float eps, int weight_per_head, int act,
                               const float* den, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads < 1 || size < 1 || act < 0 || act > 1) return LI_ERR_UNSUPPORTED;
  const size_t items = (size_t)tokens * heads;
  const int warps = 8;
  const int weight_stride = weight_per_head ? size : 0;
  const dim3 grid((unsigned)((items + warps - 1) / warps));
  // Heads of up to 512 whose rows 16-byte accesses can walk keep their row in registers.
  const size_t gate_unit = dtype == kFloat32 ? 4 : 2;
  const bool wide = size % 4 == 0 && size <= 512 && aligned16(x) && aligned16(weight) && aligned16(out) &&
                    ((uintptr_t)gate * 1) % (4 * gate_unit) == 0 && gate_stride % 4 == 0;
  if (wide) {
    const int nv = size <= 128 ? 1 : size <= 256 ? 2 : 4;
#define LI_GATED(T, NV)                                                                                                \
  return (int)launch_pdl(tokens, gated_rmsnorm_vec_kernel<T, NV>, grid, dim3(warps * 32), 0, stream, x,               \
                         (const T*)gate, gate_stride, weight, (T*)out, tokens, heads, size, eps, weight_stride, act,   \
                         den)
    if (dtype == kFloat32) {
      if (nv == 1) LI_GATED(float, 1);
      if (nv == 2) LI_GATED(float, 2);
      LI_GATED(float, 4);
    }
    if (nv == 1) LI_GATED(bf16, 1);
    if (nv == 2) LI_GATED(bf16, 2);
    LI_GATED(bf16, 4);
#undef LI_GATED
  }
  if (dtype == kFloat32)
    return (int)launch_pdl(tokens, gated_rmsnorm_kernel<float>, grid, dim3(warps * 32), 0, stream, x, (const float*)gate,
                           gate_stride, weight, (float*)out, tokens, heads, size, eps, weight_stride, act, den);
  return (int)launch_pdl(tokens, gated_rmsnorm_kernel<bf16>, grid, dim3(warps * 32), 0, stream, x, (const bf16*)gate,
                         gate_stride, weight, (bf16*)out, tokens, heads, size, eps, weight_stride, act, den);
}
