// Differential attention over a paged cache of per-token records, one thread block per (query row, head): the
// plain kernel. It serves the true 32-bit path and every shape the tensor-core kernels refuse.
//
// A head has two score maps, each a causal softmax attention of its own over the same values. Query head h
// holds [map 1 | map 2], `dim` elements each, at column h * 2 * dim of its row; KV head g = h / (heads / kv_heads)
// holds its two key maps at k_off + g * 2 * dim of a token's record and its values (vdim) at v_off + g * vdim.
// For map m of a row at position p over the keys t <= p:
//   s_t = scale * q_m . k_m,t;   s_t <- cap * tanh(s_t / cap)  (cap > 0);   a_m = softmax(s) V
// and the head's output is
//   o = a_1 - lambda * a_2;   o <- o / sqrt(mean(o^2) + eps) * out_scale
// with lambda read from device memory (one number per layer). Keys are visited in chunks whose boundaries are
// multiples of DA_CHUNK in absolute position and merged by the running (max, sum, acc) rule, so what a row
// computes depends on its own query, position and keys only. Everything is fp32 arithmetic.
#include "common.cuh"

namespace dl {

constexpr int DA_THREADS = 256;
constexpr int DA_CHUNK = 512;

template <typename T>
__global__ void __launch_bounds__(DA_THREADS)
diff_attention_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ cache, long long record, int k_off,
                      int v_off, const int* __restrict__ block_table, int max_blocks, const int* __restrict__ positions,
                      const int* __restrict__ row_slot, T* __restrict__ out, int out_stride, int n_heads, int n_kv_heads,
                      int dim, int vdim, int page_size, float scale, float softcap, const float* __restrict__ lambda,
                      float out_scale, float eps, int vec_ok) {
  __shared__ float red[33];
  __shared__ float sq[2 * 256];                // both maps of the query, fp32
  __shared__ float sp[2][DA_CHUNK];            // scores, then probabilities, of one chunk, per map
  __shared__ float part[2][DA_THREADS];        // partial weighted sums, [map][group][d]
  const int row = blockIdx.x, head = blockIdx.y;
  const int kvh = head / (n_heads / n_kv_heads);
  const int pos = positions[row];
  const int* table = block_table + static_cast<size_t>(ck_request(row_slot[row])) * max_blocks;
  const int tid = threadIdx.x;

  const T* qrow = q + static_cast<size_t>(row) * q_stride + static_cast<size_t>(head) * 2 * dim;
  for (int d = tid; d < 2 * dim; d += DA_THREADS) sq[d] = to_float(qrow[d]);
  __syncthreads();

  constexpr int V = PerVec<T>::n;
  const int groups = DA_THREADS / vdim;              // >= 1 since vdim <= 256
  const int g = tid / vdim, d = tid % vdim;          // valid when g < groups
  const size_t k_at = static_cast<size_t>(k_off) + static_cast<size_t>(kvh) * 2 * dim;
  const size_t v_at = static_cast<size_t>(v_off) + static_cast<size_t>(kvh) * vdim;

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f}, acc[2] = {0.0f, 0.0f};
  for (int c0 = 0; c0 <= pos; c0 += DA_CHUNK) {
    const int c1 = min(c0 + DA_CHUNK, pos + 1);
    float m_loc[2] = {-INFINITY, -INFINITY};
    for (int t = c0 + tid; t < c1; t += DA_THREADS) {
      const size_t slot = static_cast<size_t>(ck_page(table, t / page_size, max_blocks)) * page_size + t % page_size;
      const T* kr = cache + slot * record + k_at;
      float dot[2] = {0.0f, 0.0f};
      if (vec_ok) {
        const Vec16* kv = reinterpret_cast<const Vec16*>(kr);
        const int per_map = dim / V;
#pragma unroll
        for (int m = 0; m < 2; ++m)
          for (int i = 0; i < per_map; ++i) {
            float f[V];
            unpack<T>(kv[m * per_map + i], f);
#pragma unroll
            for (int j = 0; j < V; ++j) dot[m] = fmaf(sq[m * dim + i * V + j], f[j], dot[m]);
          }
      } else {
#pragma unroll
        for (int m = 0; m < 2; ++m)
          for (int i = 0; i < dim; ++i) dot[m] = fmaf(sq[m * dim + i], to_float(kr[m * dim + i]), dot[m]);
      }
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        float s = dot[m] * scale;
        if (softcap > 0.0f) s = softcap * tanhf(s / softcap);
        sp[m][t - c0] = s;
        m_loc[m] = fmaxf(m_loc[m], s);
      }
    }
    float corr[2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const float m_chunk = block_max(m_loc[m], red);
      const float m_new = fmaxf(m_run[m], m_chunk);       // finite: the chunk holds at least key c0
      float l_loc = 0.0f;
      for (int t = c0 + tid; t < c1; t += DA_THREADS) {
        const float p = expf(sp[m][t - c0] - m_new);
        sp[m][t - c0] = p;
        l_loc += p;
      }
      const float l_chunk = block_sum(l_loc, red);        // also orders the writes of sp before the reads below
      corr[m] = expf(m_run[m] - m_new);                   // 0 on the first chunk
      l_run[m] = l_run[m] * corr[m] + l_chunk;
      m_run[m] = m_new;
    }

    float pv[2] = {0.0f, 0.0f};
    if (g < groups) {
      for (int t = c0 + g; t < c1; t += groups) {
        const size_t slot = static_cast<size_t>(ck_page(table, t / page_size, max_blocks)) * page_size + t % page_size;
        const float v = to_float(cache[slot * record + v_at + d]);
        pv[0] = fmaf(sp[0][t - c0], v, pv[0]);
        pv[1] = fmaf(sp[1][t - c0], v, pv[1]);
      }
    }
    part[0][tid] = pv[0];
    part[1][tid] = pv[1];
    __syncthreads();
    if (tid < vdim) {
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        float sum = 0.0f;
        for (int gg = 0; gg < groups; ++gg) sum += part[m][gg * vdim + tid];
        acc[m] = acc[m] * corr[m] + sum;
      }
    }
    __syncthreads();
  }
  float o = 0.0f;
  if (tid < vdim) o = acc[0] / l_run[0] - lambda[0] * (acc[1] / l_run[1]);
  const float ss = block_sum(o * o, red);
  if (tid < vdim) {
    T* orow = out + static_cast<size_t>(row) * out_stride + static_cast<size_t>(head) * vdim;
    orow[tid] = from_float<T>(o * (1.0f / sqrtf(ss / static_cast<float>(vdim) + eps)) * out_scale);
  }
}

}  // namespace dl

// q: rows of `q_stride` elements, head h at column h * 2 * dim; out: rows of out_stride, head h at column h * vdim.
// cache: [pages, page_size, record]. dim and vdim at most 256. lambda: one float on the device.
DL_EXPORT int dl_diff_attention(int dtype, const void* q, int q_stride, const void* cache, long long record, int k_off,
                                int v_off, const int* block_table, int max_blocks, const int* positions,
                                const int* row_slot, void* out, int out_stride, int rows, int n_heads, int n_kv_heads,
                                int dim, int vdim, int page_size, float scale, float softcap, const float* lambda,
                                float out_scale, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dim <= 0 || dim > 256 || vdim <= 0 || vdim > 256 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 ||
      page_size <= 0 || n_heads > 65535)
    return DL_ERR_UNSUPPORTED;
  dim3 grid(rows, n_heads);
  const int v = dtype == 0 ? 4 : 8;
  const int vec_ok = (dim % v == 0 && record % v == 0 && k_off % v == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0) ? 1 : 0;
#define DL_LAUNCH(T)                                                                                               \
  dl::diff_attention_kernel<T><<<grid, dl::DA_THREADS, 0, stream>>>(                                               \
      static_cast<const T*>(q), q_stride, static_cast<const T*>(cache), record, k_off, v_off, block_table,         \
      max_blocks, positions, row_slot, static_cast<T*>(out), out_stride, n_heads, n_kv_heads, dim, vdim, page_size, \
      scale, softcap, lambda, out_scale, eps, vec_ok)
  if (dtype == 0) DL_LAUNCH(float);
  else if (dtype == 1) DL_LAUNCH(dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LAUNCH
  return dl::launch_status();
}
