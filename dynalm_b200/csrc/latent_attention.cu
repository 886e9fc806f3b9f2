// Latent attention over a paged cache of latents: the plain kernels.
//
// A token leaves one record in the cache: [c: R numbers, the normed latent that every head's keys and values are
// projections of | k_rot: r numbers, a rotated key part that all heads share]. With keys k_h = Uk_h c and values
// v_h = Uv_h c the score of head h is  scale * (q_h . Uk_h c + q_rot_h . k_rot) = scale * ([Uk_h^T q_h | q_rot_h] . record),
// and the head's output is Uv_h (sum_t p_t c_t): the attention itself runs on the records, with one "wide" query
// per head, and the two per-head products stand before and after it (dl_head_linear).
//
//   dl_latent_prep        per row: the normed query latent, and the row's record (normed latent, rotated key part)
//                         into its page
//   dl_head_linear        out[row, h, :] = in[row, h, :] W_h for every head (W_h stored [in, out]); optionally times
//                         sigmoid(gate[row, h, :])
//   dl_rotate_pairs       the rotated part of every head's query into the tail of its wide query
//   dl_latent_attention   one block per (row, head): softmax over the window's records with a sink in the denominator
//
// Rotation: interleaved pairs (2i, 2i+1) of the first `rot` of the r numbers turn by position * freq[i]; the angle is
// formed in double precision from a double frequency table, so that it is exact to float32 at any position.
// Norms, angles, scores, softmax and the weighted sum are float32.
#include "common.cuh"

namespace dl {

constexpr int LAT_THREADS = 256;

__device__ __forceinline__ void turn(float a, float b, int pos, double freq, float& oa, float& ob) {
  double s, c;
  sincos(static_cast<double>(pos) * freq, &s, &c);
  const float cf = static_cast<float>(c), sf = static_cast<float>(s);
  oa = a * cf - b * sf;
  ob = b * cf + a * sf;
}

// proj row: [query latent: q_rank | latent: R | key part: r | ...]. Block per row.
template <typename T>
__global__ void __launch_bounds__(LAT_THREADS)
latent_prep_kernel(const T* __restrict__ proj, int proj_stride, int q_rank, int R, int r, int rot,
                   const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                   const double* __restrict__ freq, const int* __restrict__ positions,
                   const int* __restrict__ row_slot, const int* __restrict__ block_table, int max_blocks,
                   int page_size, T* __restrict__ cq, T* __restrict__ cache) {
  __shared__ float red[33];
  const int row = blockIdx.x, tid = threadIdx.x;
  const T* pr = proj + static_cast<size_t>(row) * proj_stride;
  float ss = 0.0f;
  for (int i = tid; i < q_rank; i += LAT_THREADS) {
    const float v = to_float(pr[i]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  float inv = 1.0f / sqrtf(ss / static_cast<float>(q_rank) + eps);
  for (int i = tid; i < q_rank; i += LAT_THREADS)
    cq[static_cast<size_t>(row) * q_rank + i] = from_float<T>(to_float(pr[i]) * inv * wq[i]);
  ss = 0.0f;
  for (int i = tid; i < R; i += LAT_THREADS) {
    const float v = to_float(pr[q_rank + i]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  inv = 1.0f / sqrtf(ss / static_cast<float>(R) + eps);
  const int pos = positions[row];
  const int* table = block_table + static_cast<size_t>(ck_request(row_slot[row])) * max_blocks;
  const int page = ck_page_store(table, pos / page_size, max_blocks);
  if (page < 0) return;
  T* rec = cache + (static_cast<size_t>(page) * page_size + pos % page_size) * (R + r);
  for (int i = tid; i < R; i += LAT_THREADS) rec[i] = from_float<T>(to_float(pr[q_rank + i]) * inv * wkv[i]);
  const T* kr = pr + q_rank + R;
  for (int i = tid; i < rot / 2; i += LAT_THREADS) {
    float a, b;
    turn(to_float(kr[2 * i]), to_float(kr[2 * i + 1]), pos, freq[i], a, b);
    rec[R + 2 * i] = from_float<T>(a);
    rec[R + 2 * i + 1] = from_float<T>(b);
  }
  for (int i = rot + tid; i < r; i += LAT_THREADS) rec[R + i] = kr[i];
}

// q: [rows, H, d + r]; the last r of every head go to out[row, h, out_off .. out_off + r), the first `rot` of them
// turned. One thread per (row, head, pair or unturned element).
template <typename T>
__global__ void rotate_pairs_kernel(const T* __restrict__ q, int q_stride, int head_in, int in_off, T* __restrict__ out,
                                    int out_stride, int head_out, int out_off, int r, int rot,
                                    const double* __restrict__ freq, const int* __restrict__ positions, int rows, int H) {
  const int per = rot / 2 + (r - rot);
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * H * per) return;
  const int e = static_cast<int>(idx % per), h = static_cast<int>((idx / per) % H), row = static_cast<int>(idx / per / H);
  const T* src = q + static_cast<size_t>(row) * q_stride + static_cast<size_t>(h) * head_in + in_off;
  T* dst = out + static_cast<size_t>(row) * out_stride + static_cast<size_t>(h) * head_out + out_off;
  if (e < rot / 2) {
    float a, b;
    turn(to_float(src[2 * e]), to_float(src[2 * e + 1]), positions[row], freq[e], a, b);
    dst[2 * e] = from_float<T>(a);
    dst[2 * e + 1] = from_float<T>(b);
  } else {
    dst[rot + (e - rot / 2)] = src[rot + (e - rot / 2)];
  }
}

// out[row, h*head_out + j] = sum_i in[row, h*head_in + i] * W[h][i][j]  (j < n_out, i < n_in), optionally times
// sigmoid(gate[row, h*gate_head + j]). Block = (tile of HL_ROWS rows, head, tile of HL_THREADS outputs); a thread owns
// one output column for all rows of the tile, the tile's inputs sit in shared memory, W is read once per row tile
// with the threads of a warp on consecutive columns. The sum runs over i in order: it depends on the row alone.
constexpr int HL_ROWS = 8;
constexpr int HL_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(HL_THREADS)
head_linear_kernel(const T* __restrict__ in, int in_stride, int head_in, int n_in, const T* __restrict__ W, int n_out,
                   T* __restrict__ out, int out_stride, int head_out, const T* __restrict__ gate, int gate_stride,
                   int gate_head, int rows) {
  extern __shared__ float sin_[];                 // [HL_ROWS][n_in]
  const int row0 = blockIdx.x * HL_ROWS, h = blockIdx.y, j = blockIdx.z * HL_THREADS + threadIdx.x;
  const int nr = min(HL_ROWS, rows - row0);
  for (int i = threadIdx.x; i < HL_ROWS * n_in; i += HL_THREADS) {
    const int rr = i / n_in, c = i % n_in;
    sin_[i] = rr < nr ? to_float(in[static_cast<size_t>(row0 + rr) * in_stride + static_cast<size_t>(h) * head_in + c]) : 0.0f;
  }
  __syncthreads();
  if (j >= n_out) return;
  const T* w = W + static_cast<size_t>(h) * n_in * n_out + j;
  float acc[HL_ROWS];
#pragma unroll
  for (int rr = 0; rr < HL_ROWS; ++rr) acc[rr] = 0.0f;
  for (int i = 0; i < n_in; ++i) {
    const float wv = to_float(w[static_cast<size_t>(i) * n_out]);
#pragma unroll
    for (int rr = 0; rr < HL_ROWS; ++rr) acc[rr] = fmaf(sin_[rr * n_in + i], wv, acc[rr]);
  }
#pragma unroll
  for (int rr = 0; rr < HL_ROWS; ++rr) {
    if (rr < nr) {
      float v = acc[rr];
      if (gate) {
        // the product is rounded to the storage type first, as when it is a tensor of its own
        v = to_float(from_float<T>(v));
        const float g = to_float(gate[static_cast<size_t>(row0 + rr) * gate_stride + static_cast<size_t>(h) * gate_head + j]);
        v *= 1.0f / (1.0f + expf(-g));
      }
      out[static_cast<size_t>(row0 + rr) * out_stride + static_cast<size_t>(h) * head_out + j] = from_float<T>(v);
    }
  }
}

// One block per (row, head). qw: the wide query [R + r] of the head; the keys are the records of positions
// [lo, pos], lo = window > 0 ? max(0, pos - window + 1) : 0, visited in chunks at absolute multiples of LAT_CHUNK.
// out[row, h, 0..R) = sum_t p_t c_t / (sum_t p_t + exp(sink_h - max)).
constexpr int LAT_CHUNK = 512;
constexpr int LAT_MAX_DIMS = 4;                   // R up to LAT_MAX_DIMS * LAT_THREADS

template <typename T>
__global__ void __launch_bounds__(LAT_THREADS)
latent_attention_kernel(const T* __restrict__ qw, int q_stride, const T* __restrict__ cache, const int* __restrict__ block_table,
                        int max_blocks, const int* __restrict__ positions, const int* __restrict__ row_slot,
                        const float* __restrict__ sink, T* __restrict__ out, int out_stride, int R, int r, int page_size,
                        float scale, int window) {
  extern __shared__ float sq[];                   // the wide query, float32 [R + r]
  __shared__ float red[33];
  __shared__ float sp[LAT_CHUNK];
  const int row = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int RW = R + r;
  const int pos = positions[row];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int* table = block_table + static_cast<size_t>(ck_request(row_slot[row])) * max_blocks;
  const T* qr = qw + static_cast<size_t>(row) * q_stride + static_cast<size_t>(head) * RW;
  for (int i = tid; i < RW; i += LAT_THREADS) sq[i] = to_float(qr[i]);
  __syncthreads();

  float m_run = -INFINITY, l_run = 0.0f;
  float acc[LAT_MAX_DIMS];
#pragma unroll
  for (int k = 0; k < LAT_MAX_DIMS; ++k) acc[k] = 0.0f;
  for (int c0 = (lo / LAT_CHUNK) * LAT_CHUNK; c0 <= pos; c0 += LAT_CHUNK) {
    const int c1 = min(c0 + LAT_CHUNK, pos + 1);
    // scores: a warp per key, its lanes over the record, summed in a fixed order
    for (int t = c0 + warp; t < c1; t += LAT_THREADS / 32) {
      float s = -INFINITY;
      if (t >= lo) {
        const T* rec = cache + (static_cast<size_t>(ck_page(table, t / page_size, max_blocks)) * page_size + t % page_size) * RW;
        float dot = 0.0f;
        for (int i = lane; i < RW; i += 32) dot = fmaf(sq[i], to_float(rec[i]), dot);
        s = warp_sum(dot) * scale;
      }
      if (lane == 0) sp[t - c0] = s;
    }
    __syncthreads();
    float m_loc = -INFINITY;
    for (int t = c0 + tid; t < c1; t += LAT_THREADS) m_loc = fmaxf(m_loc, sp[t - c0]);
    const float m_new = fmaxf(m_run, block_max(m_loc, red));       // finite: the chunk holds key max(lo, c0)
    float l_loc = 0.0f;
    for (int t = c0 + tid; t < c1; t += LAT_THREADS) {
      const float p = expf(sp[t - c0] - m_new);                   // exp(-inf) = 0 for keys before lo
      sp[t - c0] = p;
      l_loc += p;
    }
    const float l_chunk = block_sum(l_loc, red);                  // also orders the writes of sp before the reads below
    const float corr = expf(m_run - m_new);                       // 0 on the first chunk
    l_run = l_run * corr + l_chunk;
    m_run = m_new;
#pragma unroll
    for (int k = 0; k < LAT_MAX_DIMS; ++k) acc[k] *= corr;
    for (int t = max(c0, lo); t < c1; ++t) {
      const T* rec = cache + (static_cast<size_t>(ck_page(table, t / page_size, max_blocks)) * page_size + t % page_size) * RW;
      const float p = sp[t - c0];
#pragma unroll
      for (int k = 0; k < LAT_MAX_DIMS; ++k) {
        const int d = tid + k * LAT_THREADS;
        if (d < R) acc[k] = fmaf(p, to_float(rec[d]), acc[k]);
      }
    }
    __syncthreads();
  }
  float den = l_run, keep = 1.0f;
  if (sink) {
    const float sk = sink[head];
    const float m_all = fmaxf(m_run, sk);
    keep = expf(m_run - m_all);
    den = l_run * keep + expf(sk - m_all);
  }
  T* orow = out + static_cast<size_t>(row) * out_stride + static_cast<size_t>(head) * R;
#pragma unroll
  for (int k = 0; k < LAT_MAX_DIMS; ++k) {
    const int d = tid + k * LAT_THREADS;
    if (d < R) orow[d] = from_float<T>(acc[k] * keep / den);
  }
}

}  // namespace dl

DL_EXPORT int dl_latent_prep(int dtype, const void* proj, int proj_stride, int q_rank, int R, int r, int rot, const float* wq,
                             const float* wkv, float eps, const double* freq, const int* positions, const int* row_slot,
                             const int* block_table, int max_blocks, int page_size, void* cq, void* cache, int rows,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (q_rank <= 0 || R <= 0 || r < 0 || rot < 0 || rot > r || rot % 2 != 0 || page_size <= 0) return DL_ERR_UNSUPPORTED;
#define DL_LAUNCH(T)                                                                                                   \
  dl::latent_prep_kernel<T><<<rows, dl::LAT_THREADS, 0, stream>>>(static_cast<const T*>(proj), proj_stride, q_rank, R, r, rot, \
                                                                  wq, wkv, eps, freq, positions, row_slot, block_table, \
                                                                  max_blocks, page_size, static_cast<T*>(cq), static_cast<T*>(cache))
  if (dtype == 0) DL_LAUNCH(float);
  else if (dtype == 1) DL_LAUNCH(dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LAUNCH
  return dl::launch_status();
}

DL_EXPORT int dl_rotate_pairs(int dtype, const void* q, int q_stride, int head_in, int in_off, void* out, int out_stride,
                              int head_out, int out_off, int r, int rot, const double* freq, const int* positions, int rows,
                              int H, cudaStream_t stream) {
  if (rows <= 0 || H <= 0 || r <= 0) return 0;
  if (rot < 0 || rot > r || rot % 2 != 0) return DL_ERR_UNSUPPORTED;
  const size_t n = static_cast<size_t>(rows) * H * (rot / 2 + (r - rot));
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n + threads - 1) / threads);
#define DL_LAUNCH(T)                                                                                                  \
  dl::rotate_pairs_kernel<T><<<blocks, threads, 0, stream>>>(static_cast<const T*>(q), q_stride, head_in, in_off,     \
                                                             static_cast<T*>(out), out_stride, head_out, out_off, r, rot, \
                                                             freq, positions, rows, H)
  if (dtype == 0) DL_LAUNCH(float);
  else if (dtype == 1) DL_LAUNCH(dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LAUNCH
  return dl::launch_status();
}

// W: [H, n_in, n_out] contiguous. gate may be null.
DL_EXPORT int dl_head_linear(int dtype, const void* in, int in_stride, int head_in, int n_in, const void* W, int n_out,
                             void* out, int out_stride, int head_out, const void* gate, int gate_stride, int gate_head,
                             int rows, int H, cudaStream_t stream) {
  if (rows <= 0 || H <= 0 || n_out <= 0) return 0;
  const size_t smem = sizeof(float) * dl::HL_ROWS * static_cast<size_t>(n_in);
  if (n_in <= 0 || H > 65535 || smem > 160 * 1024) return DL_ERR_UNSUPPORTED;
  dim3 grid((rows + dl::HL_ROWS - 1) / dl::HL_ROWS, H, (n_out + dl::HL_THREADS - 1) / dl::HL_THREADS);
#define DL_LAUNCH(T)                                                                                                    \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(dl::head_linear_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    dl::head_linear_kernel<T><<<grid, dl::HL_THREADS, smem, stream>>>(static_cast<const T*>(in), in_stride, head_in, n_in, \
                                                                      static_cast<const T*>(W), n_out, static_cast<T*>(out), \
                                                                      out_stride, head_out, static_cast<const T*>(gate), \
                                                                      gate_stride, gate_head, rows);                    \
  } while (0)
  if (dtype == 0) DL_LAUNCH(float);
  else if (dtype == 1) DL_LAUNCH(dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LAUNCH
  return dl::launch_status();
}

// qw: [rows, H, R + r] wide queries; cache: [pages, page_size, R + r]; out: [rows, H, R].
DL_EXPORT int dl_latent_attention(int dtype, const void* qw, int q_stride, const void* cache, const int* block_table,
                                  int max_blocks, const int* positions, const int* row_slot, const float* sink, void* out,
                                  int out_stride, int rows, int H, int R, int r, int page_size, float scale, int window,
                                  cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || H > 65535 || R <= 0 || R > dl::LAT_MAX_DIMS * dl::LAT_THREADS || r < 0 || page_size <= 0 || window < 0)
    return DL_ERR_UNSUPPORTED;
  const size_t smem = sizeof(float) * static_cast<size_t>(R + r);
  if (smem > 40 * 1024) return DL_ERR_UNSUPPORTED;
  dim3 grid(rows, H);
#define DL_LAUNCH(T)                                                                                                  \
  dl::latent_attention_kernel<T><<<grid, dl::LAT_THREADS, smem, stream>>>(static_cast<const T*>(qw), q_stride,         \
                                                                          static_cast<const T*>(cache), block_table,   \
                                                                          max_blocks, positions, row_slot, sink,       \
                                                                          static_cast<T*>(out), out_stride, R, r,      \
                                                                          page_size, scale, window)
  if (dtype == 0) DL_LAUNCH(float);
  else if (dtype == 1) DL_LAUNCH(dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LAUNCH
  return dl::launch_status();
}
