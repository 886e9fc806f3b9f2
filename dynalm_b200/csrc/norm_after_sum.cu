// RMSNorm AFTER the residual sum, for layers that norm what they have just added up:
//
//   v    = alpha * x[r] + s * delta[r]          (s: a per-channel scale of the sublayer's result, or none)
//   x[r] = v / sqrt(mean(v^2) + eps) * w        (the float32 residual stream now IS the normed row)
//   out[r] = x[r] in the compute dtype          (what the next sublayer's matrix products read; optional)
//
// delta may come as `parts` split-K partial sums, `part_stride` elements apart, added in index order. Everything is
// float32; the sum of squares is a fixed-order tree over the block. Also here: the float32 -> compute dtype copy of
// rows, for the first layer of such a model (its input is the embedding, which nothing has normed).
#include "common.cuh"

namespace dl {

template <typename TD>
__device__ __forceinline__ float sum_parts(const TD* d0, size_t i, int parts, size_t part_stride) {
  float d = to_float(d0[i]);
  for (int p = 1; p < parts; ++p) d += to_float(d0[p * part_stride + i]);
  return d;
}

constexpr int NAS_THREADS = 256;

// Any width: the summed row is parked in x between the two passes.
template <typename TO, typename TD>
__global__ void __launch_bounds__(NAS_THREADS)
norm_after_sum_kernel(float* __restrict__ x, const TD* __restrict__ delta, int parts, size_t part_stride,
                      const float* __restrict__ delta_scale, float alpha, const float* __restrict__ w, float eps,
                      TO* __restrict__ out, int width) {
  __shared__ float red[33];
  const size_t base = static_cast<size_t>(blockIdx.x) * width;
  float* xr = x + base;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < width; i += NAS_THREADS) {
    float d = sum_parts(delta, base + i, parts, part_stride);
    if (delta_scale) d *= delta_scale[i];
    const float v = fmaf(alpha, xr[i], d);
    xr[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  for (int i = threadIdx.x; i < width; i += NAS_THREADS) {
    const float y = xr[i] * inv * w[i];
    xr[i] = y;
    if (out) out[base + i] = from_float<TO>(y);
  }
}

template <typename T> __device__ __forceinline__ float4 ld4(const T* p);
template <> __device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ld4<bf16>(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                     __uint_as_float(u.y & 0xffff0000u));
}
template <typename T> __device__ __forceinline__ void st4(T* p, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4<bf16>(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// Widths that are a multiple of 4 and at most NV * 1024: the row stays in registers, one pass over memory with
// 16-byte accesses (8-byte for a bfloat16 delta), every load of a thread issued before its first use.
template <typename TO, typename TD, int NV>
__global__ void __launch_bounds__(NAS_THREADS)
norm_after_sum_vec_kernel(float* __restrict__ x, const TD* __restrict__ delta, int parts, size_t part_stride,
                          const float* __restrict__ delta_scale, float alpha, const float* __restrict__ w, float eps,
                          TO* __restrict__ out, int width) {
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const size_t base = static_cast<size_t>(blockIdx.x) * width;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v[NV], d[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * NAS_THREADS + threadIdx.x) * 4;
    v[i] = c < width ? ld4<float>(x + base + c) : zero;
    d[i] = c < width ? ld4<TD>(delta + base + c) : zero;
  }
  for (int p = 1; p < parts; ++p) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * NAS_THREADS + threadIdx.x) * 4;
      const float4 e = c < width ? ld4<TD>(delta + p * part_stride + base + c) : zero;
      d[i].x += e.x; d[i].y += e.y; d[i].z += e.z; d[i].w += e.w;
    }
  }
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * NAS_THREADS + threadIdx.x) * 4;
    if (delta_scale && c < width) {
      const float4 s = ld4<float>(delta_scale + c);
      d[i].x *= s.x; d[i].y *= s.y; d[i].z *= s.z; d[i].w *= s.w;
    }
    v[i].x = fmaf(alpha, v[i].x, d[i].x); v[i].y = fmaf(alpha, v[i].y, d[i].y);
    v[i].z = fmaf(alpha, v[i].z, d[i].z); v[i].w = fmaf(alpha, v[i].w, d[i].w);
    ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * NAS_THREADS + threadIdx.x) * 4;
    if (c < width) {
      const float4 g = ld4<float>(w + c);
      const float4 y = make_float4(v[i].x * inv * g.x, v[i].y * inv * g.y, v[i].z * inv * g.z, v[i].w * inv * g.w);
      st4<float>(x + base + c, y);
      if (out) st4<TO>(out + base + c, y);
    }
  }
}

template <typename TO>
__global__ void cast_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_float<TO>(x[i]);
}

template <typename TO, typename TD>
int norm_after_sum_launch(float* x, const void* delta, int parts, long long part_stride, const float* delta_scale,
                          float alpha, const float* w, float eps, void* out, int rows, int width, cudaStream_t stream) {
  const TD* d = static_cast<const TD*>(delta);
  TO* o = static_cast<TO*>(out);
  const size_t ps = static_cast<size_t>(part_stride);
  const bool aligned = width % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(delta) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
                       (delta_scale == nullptr || (reinterpret_cast<uintptr_t>(delta_scale) & 15) == 0) &&
                       (out == nullptr || (reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                       (part_stride * static_cast<long long>(sizeof(TD))) % 16 == 0;
#define DL_NAS(NV)                                                                                              \
  return launch(norm_after_sum_vec_kernel<TO, TD, NV>, dim3(rows), dim3(NAS_THREADS), 0, stream, x, d, parts, ps, \
                delta_scale, alpha, w, eps, o, width)
  if (aligned && width <= 1024) DL_NAS(1);
  if (aligned && width <= 2048) DL_NAS(2);
  if (aligned && width <= 4096) DL_NAS(4);
  if (aligned && width <= 8192) DL_NAS(8);
#undef DL_NAS
  norm_after_sum_kernel<TO, TD><<<rows, NAS_THREADS, 0, stream>>>(x, d, parts, ps, delta_scale, alpha, w, eps, o, width);
  return launch_status();
}

}  // namespace dl

// x: float32 [rows, width], replaced by the normed rows. delta: [rows, width] of `delta_dtype` (0 float32, 1
// bfloat16), or `parts` such arrays `part_stride` elements apart. delta_scale: float32 [width] or null. out:
// [rows, width] of `out_dtype`, or null.
DL_EXPORT int dl_norm_after_sum(int out_dtype, int delta_dtype, float* x, const void* delta, int parts,
                                long long part_stride, const float* delta_scale, float alpha, const float* w, float eps,
                                void* out, int rows, int width, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (width <= 0 || parts <= 0 || delta == nullptr) return DL_ERR_UNSUPPORTED;
  if (out_dtype == 0 && delta_dtype == 0)
    return dl::norm_after_sum_launch<float, float>(x, delta, parts, part_stride, delta_scale, alpha, w, eps, out, rows, width, stream);
  if (out_dtype == 1 && delta_dtype == 1)
    return dl::norm_after_sum_launch<dl::bf16, dl::bf16>(x, delta, parts, part_stride, delta_scale, alpha, w, eps, out, rows, width, stream);
  if (out_dtype == 1 && delta_dtype == 0)
    return dl::norm_after_sum_launch<dl::bf16, float>(x, delta, parts, part_stride, delta_scale, alpha, w, eps, out, rows, width, stream);
  return DL_ERR_UNSUPPORTED;
}

// out[i] = x[i] in `out_dtype` over n contiguous elements.
DL_EXPORT int dl_cast_rows(int out_dtype, const float* x, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((static_cast<size_t>(n) + threads - 1) / threads);
  if (out_dtype == 1) dl::cast_rows_kernel<dl::bf16><<<blocks, threads, 0, stream>>>(x, static_cast<dl::bf16*>(out), static_cast<size_t>(n));
  else if (out_dtype == 0) dl::cast_rows_kernel<float><<<blocks, threads, 0, stream>>>(x, static_cast<float*>(out), static_cast<size_t>(n));
  else return DL_ERR_UNSUPPORTED;
  return dl::launch_status();
}
