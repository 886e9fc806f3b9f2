// Per-head RMS norm of queries and keys, a position-dependent query temperature, and the write of the
// normalised keys and the values into a paged cache of per-token records: what an attention mixer without a
// rotation does between its projections and its scores (the counterpart of rope_cache.cu for such mixers).
//
// A row of `qkv` is [q units | k units | values]: n_q_units + n_k_units "units" of `dim` elements each (a unit is
// one head, or one score map of one head) followed by v_width value elements. For a unit x:
//   y = x / sqrt(mean(x^2) + eps) * w            w: float32 [dim], one for the queries and one for the keys,
//                                                 shared by all units
//   queries only, at position p:  y *= 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)     (temp_every > 0)
// Queries are normalised in place. Keys go, normalised, to the token's record in the cache at k_off + unit * dim,
// values as they are to v_off + e; the record of position p of the request in slot s is
// cache[(block_table[s][p / page_size] * page_size + p % page_size) * record]. A layer that reads another
// layer's cache passes write_cache = 0 and only its queries are touched.
//
// All arithmetic is fp32 whatever the storage type; a unit is one warp's work and its sum of squares is a warp
// tree, so a row's result depends on nothing but the row.
#include "common.cuh"

namespace dl {

constexpr int QKN_WARPS = 4;
constexpr int QKN_VCHUNK = 256;      // value elements one warp copies

template <typename T>
__global__ void __launch_bounds__(QKN_WARPS * 32)
qk_norm_cache_kernel(T* __restrict__ qkv, int stride, const int* __restrict__ positions, const int* __restrict__ row_slot,
                     const int* __restrict__ block_table, int max_blocks, T* __restrict__ cache, long long record,
                     int k_off, int v_off, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                     float temp_coef, int temp_every, int n_q_units, int n_k_units, int dim, int v_width,
                     int page_size, int write_cache) {
  const int row = blockIdx.x;
  const int unit = blockIdx.y * QKN_WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int v_units = write_cache ? (v_width + QKN_VCHUNK - 1) / QKN_VCHUNK : 0;
  const int k_units = write_cache ? n_k_units : 0;
  if (unit >= n_q_units + k_units + v_units) return;
  T* xr = qkv + static_cast<size_t>(row) * stride;
  const int pos = positions[row];
  T* rec = nullptr;
  if (unit >= n_q_units) {
    const int* table = block_table + static_cast<size_t>(ck_request(row_slot[row])) * max_blocks;
    const int page = ck_page_store(table, pos / page_size, max_blocks);
    if (page < 0) return;
    rec = cache + (static_cast<size_t>(page) * page_size + pos % page_size) * record;
  }
  if (unit >= n_q_units + k_units) {
    // values: a plain copy
    const int e0 = (unit - n_q_units - k_units) * QKN_VCHUNK;
    const T* src = xr + static_cast<size_t>(n_q_units + n_k_units) * dim;
    for (int e = e0 + lane; e < min(e0 + QKN_VCHUNK, v_width); e += 32) rec[v_off + e] = src[e];
    return;
  }
  const bool is_q = unit < n_q_units;
  T* x = xr + static_cast<size_t>(unit) * dim;
  float ss = 0.0f;
  for (int d = lane; d < dim; d += 32) {
    const float v = to_float(x[d]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  float mul = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
  const float* w = is_q ? q_w : k_w;
  T* dst = is_q ? x : rec + k_off + static_cast<size_t>(unit - n_q_units) * dim;
  float temp = 1.0f;
  if (is_q && temp_every > 0) temp = 1.0f + temp_coef * logf(static_cast<float>((pos + 1) / temp_every) + 1.0f);
  for (int d = lane; d < dim; d += 32) dst[d] = from_float<T>(to_float(x[d]) * mul * w[d] * temp);
}

// The same with 16 bytes per thread: a unit is `tg` neighbouring lanes of a warp (tg = dim / elements per vector, a
// power of two up to 32), its sum of squares a butterfly over those lanes. A row's vectors are numbered through
// queries, keys and values.
template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_cache_vec_kernel(T* __restrict__ qkv, int stride, const int* __restrict__ positions, const int* __restrict__ row_slot,
                         const int* __restrict__ block_table, int max_blocks, T* __restrict__ cache, long long record,
                         int k_off, int v_off, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                         float temp_coef, int temp_every, int n_q_units, int n_k_units, int dim, int v_width,
                         int page_size, int write_cache, int tg) {
  constexpr int V = PerVec<T>::n;
  const int row = blockIdx.x;
  const int vec = blockIdx.y * blockDim.x + threadIdx.x;
  const int nq = n_q_units * tg, nk = write_cache ? n_k_units * tg : 0, nv = write_cache ? v_width / V : 0;
  const bool live = vec < nq + nk + nv;
  T* xr = qkv + static_cast<size_t>(row) * stride;
  Vec16 raw;
  raw.raw = make_uint4(0u, 0u, 0u, 0u);
  if (live) raw = *reinterpret_cast<const Vec16*>(xr + static_cast<size_t>(vec) * V);
  float f[V];
  unpack<T>(raw, f);
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < V; ++j) ss = fmaf(f[j], f[j], ss);
  for (int o = tg >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (!live) return;
  const int pos = positions[row];
  T* rec = nullptr;
  if (vec >= nq) {
    const int* table = block_table + static_cast<size_t>(ck_request(row_slot[row])) * max_blocks;
    const int page = ck_page_store(table, pos / page_size, max_blocks);
    if (page < 0) return;
    rec = cache + (static_cast<size_t>(page) * page_size + pos % page_size) * record;
  }
  if (vec >= nq + nk) {
    *reinterpret_cast<Vec16*>(rec + v_off + static_cast<size_t>(vec - nq - nk) * V) = raw;
    return;
  }
  const bool is_q = vec < nq;
  const float mul = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
  const float* w = (is_q ? q_w : k_w) + (vec % tg) * V;
  float temp = 1.0f;
  if (is_q && temp_every > 0) temp = 1.0f + temp_coef * logf(static_cast<float>((pos + 1) / temp_every) + 1.0f);
#pragma unroll
  for (int j = 0; j < V; ++j) f[j] = f[j] * mul * w[j] * temp;
  T* dst = is_q ? xr + static_cast<size_t>(vec) * V : rec + k_off + static_cast<size_t>(vec - nq) * V;
  *reinterpret_cast<Vec16*>(dst) = pack<T>(f);
}

}  // namespace dl

// dtype: 0 = float32, 1 = bfloat16 (qkv and the cache alike). q_w, k_w: float32 [dim] (k_w may be null when
// write_cache is 0). record: elements per token of the cache; k_off, v_off: where keys and values begin in it.
DL_EXPORT int dl_qk_norm_cache_write(int dtype, void* qkv, int stride, const int* positions, const int* row_slot,
                                     const int* block_table, int max_blocks, void* cache, long long record, int k_off,
                                     int v_off, const float* q_w, const float* k_w, float eps, float temp_coef,
                                     int temp_every, int rows, int n_q_units, int n_k_units, int dim, int v_width,
                                     int page_size, int write_cache, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dim <= 0 || n_q_units < 0 || n_k_units < 0 || v_width < 0 || page_size <= 0) return DL_ERR_UNSUPPORTED;
  const int units = n_q_units + (write_cache ? n_k_units + (v_width + dl::QKN_VCHUNK - 1) / dl::QKN_VCHUNK : 0);
  if (units <= 0) return 0;
  // 16 bytes per thread where units, rows and records allow it
  const int vlen = dtype == 0 ? 4 : 8;
  const int tg = dim / vlen;
  if ((dtype == 0 || dtype == 1) && dim % vlen == 0 && tg >= 1 && tg <= 32 && (tg & (tg - 1)) == 0 && stride % vlen == 0 &&
      (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 &&
      (!write_cache || (record % vlen == 0 && k_off % vlen == 0 && v_off % vlen == 0 && v_width % vlen == 0 &&
                        (reinterpret_cast<uintptr_t>(cache) & 15) == 0))) {
    const int total = n_q_units * tg + (write_cache ? n_k_units * tg + v_width / vlen : 0);
    const int threads = total <= 128 ? 128 : 256;
    dim3 vgrid(rows, (total + threads - 1) / threads);
    if (vgrid.y <= 65535) {
#define DL_VEC(T)                                                                                                        \
  dl::qk_norm_cache_vec_kernel<T><<<vgrid, threads, 0, stream>>>(                                                       \
      static_cast<T*>(qkv), stride, positions, row_slot, block_table, max_blocks, static_cast<T*>(cache), record, k_off, \
      v_off, q_w, k_w, eps, temp_coef, temp_every, n_q_units, n_k_units, dim, v_width, page_size, write_cache, tg)
      if (dtype == 0) DL_VEC(float);
      else DL_VEC(dl::bf16);
#undef DL_VEC
      return dl::launch_status();
    }
  }
  dim3 grid(rows, (units + dl::QKN_WARPS - 1) / dl::QKN_WARPS);
  if (grid.y > 65535) return DL_ERR_UNSUPPORTED;
#define DL_LAUNCH(T)                                                                                                  \
  dl::qk_norm_cache_kernel<T><<<grid, dl::QKN_WARPS * 32, 0, stream>>>(                                               \
      static_cast<T*>(qkv), stride, positions, row_slot, block_table, max_blocks, static_cast<T*>(cache), record,     \
      k_off, v_off, q_w, k_w, eps, temp_coef, temp_every, n_q_units, n_k_units, dim, v_width, page_size, write_cache)
  if (dtype == 0) DL_LAUNCH(float);
  else if (dtype == 1) DL_LAUNCH(dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LAUNCH
  return dl::launch_status();
}
