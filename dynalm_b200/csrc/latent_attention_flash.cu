// Latent attention over a paged cache of records on bf16 tensor cores (mma.sync m16n8k16), softmax in fp32.
//
// Every head's wide query [Uk_h^T q_h | rot(q_rot_h)] is scored against the same records [c | k_rot] (see
// latent_attention.cu), and the softmax weights sum the records' latents: attention with ONE key/value head whose
// keys are R + r wide and whose values are the first R numbers of the keys. So the rows of the tensor-core tile are
// query UNITS, a unit being (query row, head): a block takes QR consecutive rows of one request times HG heads, 32
// units at most, and walks the keys its rows may see, 64 at a time, double-buffered with cp.async; a record is read
// once for all 32 units.
//
//   scores   warp w takes units 16 (w & 1) .. +15 and keys 16 (w >> 1) .. +15 of the tile: S = Q K^T over all R + r
//            numbers, Q from shared memory (it is too wide for registers)
//   softmax  per-unit maxima and sums of the four warps that share a unit go through shared memory; every thread keeps
//            the running maximum and sum of the four units whose output it holds; P is rounded to bf16
//   output   warp w holds all 32 units times columns [w R/8, (w + 1) R/8) of O and adds P V, V = the latents of the tile
//
// Key tiles begin at multiples of 64 in absolute position, so a unit's arithmetic does not depend on where its
// request was cut or what else the step holds. A unit at position p sees keys t with 0 <= p - t < window (window 0:
// all t <= p); the sink of its head enters the denominator at the end. Exponentials are ex2.approx of scores scaled
// by log2(e). R and r are run-time multiples of 8, R at most 512; every size comes with the launch.
#include "tcgen05.cuh"

namespace dl {

constexpr int LF_M = 32;         // units per block
constexpr int LF_KT = 64;        // keys per tile
constexpr int LF_THREADS = 256;
constexpr int LF_PS = LF_KT + 8; // row stride of P in shared memory (bf16)
constexpr float LF_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void lf_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void lf_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void lf_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float lf_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t lf_pack(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ void lf_cp16(uint32_t smem, const void* gmem, bool valid) {
  const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void lf_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void lf_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

struct LatentFlashParams {
  const bf16* qw;
  int q_stride;
  const bf16* cache;
  const int* block_table;
  int max_blocks;
  const int* tiles;        // [n][4] = (request slot, first row of the step, rows, first position)
  const float* sink;
  bf16* out;
  int out_stride;
  int H, R, r, page_size, window, HG;      // HG heads of QR = 32 / HG rows to a block (one row when HG = 32)
  float scale;
  int* status;             // (bulk copies) receives LF_ERR_COPY when a wait for a tile's records gives up
  int parts;               // > 1: the key tiles of every query tile are dealt over this many blocks (blockIdx.z), which
  float* scratch;          // leave (max, sum, O) per unit in scratch [row, head, part, R + 2] for the merge kernel
};

// Records of keys [t0, t0 + 64) into a stage: a warp takes 8 keys, its lanes a key's 16-byte pieces. Keys outside
// [lo, hi] are zero-filled (their weights are zero, and zero times what a stage held before must stay zero).
__device__ __forceinline__ void lf_load_keys(const LatentFlashParams& p, const int* table, bf16* stage, int RS, int RW, int t0,
                                             int lo, int hi, int warp, int lane) {
  const int pieces = RW / 8;
#pragma unroll 1
  for (int i = 0; i < 8; ++i) {
    const int key = warp * 8 + i, t = t0 + key;
    const bool valid = t >= lo && t <= hi;
    const bf16* rec = p.cache;
    if (valid) {
      const int page = ck_page(table, t / p.page_size, p.max_blocks);
      rec += (static_cast<size_t>(page) * p.page_size + t % p.page_size) * RW;
    }
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(stage + static_cast<size_t>(key) * RS));
    for (int c = lane; c < pieces; c += 32) lf_cp16(dst + c * 16, rec + c * 8, valid);
  }
}

// The same with ONE bulk copy per record (cp.async.bulk, completion counted in bytes on the stage's mbarrier) instead of
// 16-byte pieces: 64 copy instructions a tile instead of several thousand, issued by the first warp, each lane its keys
// `lane` and `lane + 32`. Rows of keys outside [lo, hi] are zeroed by ordinary stores.
__device__ __forceinline__ void lf_load_keys_bulk(const LatentFlashParams& p, const int* table, bf16* stage, int RS, int RW,
                                                  int t0, int lo, int hi, int lane, uint64_t* bar) {
  const uint32_t bytes = static_cast<uint32_t>(RW) * 2u;
  const bf16* src[2];
  bool valid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int t = t0 + lane + 32 * i;
    valid[i] = t >= lo && t <= hi;
    src[i] = p.cache;
    if (valid[i]) {
      const int page = ck_page(table, t / p.page_size, p.max_blocks);
      src[i] += (static_cast<size_t>(page) * p.page_size + t % p.page_size) * RW;
    }
  }
  const int n_valid = __popc(__ballot_sync(0xffffffffu, valid[0])) + __popc(__ballot_sync(0xffffffffu, valid[1]));
  // ordinary stores into this stage (zeroed rows of an earlier tile) come before the copies that write it now
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(n_valid) * bytes);      // (one arrival: the phase ends when the bytes are in)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    bf16* dst = stage + static_cast<size_t>(lane + 32 * i) * RS;
    if (valid[i]) {
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(smem_u32(dst)), "l"(src[i]), "r"(bytes), "r"(smem_u32(bar)) : "memory");
    } else {
      for (int c = 0; c < RW; c += 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

constexpr int LF_ERR_COPY = 31;    // status code: a tile's records did not arrive within about a second

// NT: 8-column tiles of O per warp (R <= 64 NT). BULK: records by bulk copies and mbarriers instead of cp.async pieces.
template <int NT, bool BULK>
__global__ void __launch_bounds__(LF_THREADS, 1)
latent_attention_flash_kernel(const LatentFlashParams p) {
  __shared__ __align__(8) uint64_t lf_bar[2];
  __shared__ int lf_abort;
  extern __shared__ __align__(16) unsigned char lf_smem[];
  const int RW = p.R + p.r;
  const int RWp = (RW + 15) & ~15;
  const int RS = RWp + 8;                                   // row stride of Q and K (bf16): rows 16 bytes apart modulo 128
  bf16* sQ = reinterpret_cast<bf16*>(lf_smem);              // [32][RS]
  bf16* sK = sQ + LF_M * RS;                                // [2][64][RS]
  bf16* sP = sK + 2 * LF_KT * RS;                           // [32][LF_PS]
  float* sPMax = reinterpret_cast<float*>(sP + LF_M * LF_PS);   // [4][32]
  float* sPSum = sPMax + 4 * LF_M;                          // [4][32]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, q4 = lane & 3;
  if (BULK && tid == 0) {
    mbar_init(&lf_bar[0], 1);
    mbar_init(&lf_bar[1], 1);
    lf_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();
  pdl_trigger();
  const int4 tile = ck_tile(reinterpret_cast<const int4*>(p.tiles)[blockIdx.x]);
  const int slot = tile.x, row0 = tile.y, rows = tile.z, pos0 = tile.w;
  const int h0 = blockIdx.y * p.HG;
  const int heads = min(p.HG, p.H - h0);                    // heads of this block
  if (rows <= 0) return;
  if (BULK) __syncthreads();                                 // the barriers are initialised
  const int* table = p.block_table + static_cast<size_t>(slot) * p.max_blocks;
  const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;       // the oldest key the first row sees
  const int hi = pos0 + rows - 1;                                       // the newest key the last row sees
  const bool two = rows * p.HG > 16;                        // units 16 .. 31 hold anything

  // unit u = (row u / HG of the tile, head h0 + u % HG)
  for (int i = tid; i < LF_M * (RS / 8); i += LF_THREADS) {
    const int u = i / (RS / 8), c = (i % (RS / 8)) * 8;
    const int ur = u / p.HG, uh = u % p.HG;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (ur < rows && uh < heads && c < RW)
      v = *reinterpret_cast<const uint4*>(p.qw + static_cast<size_t>(row0 + ur) * p.q_stride + static_cast<size_t>(h0 + uh) * RW + c);
    *reinterpret_cast<uint4*>(sQ + static_cast<size_t>(u) * RS + c) = v;
  }
  // the columns of K behind the record are never loaded: zero once
  for (int i = tid; i < 2 * LF_KT * ((RS - RW) / 8); i += LF_THREADS) {
    const int k = i / ((RS - RW) / 8), c = RW + (i % ((RS - RW) / 8)) * 8;
    *reinterpret_cast<uint4*>(sK + static_cast<size_t>(k) * RS + c) = make_uint4(0u, 0u, 0u, 0u);
  }
  for (int i = tid; i < 4 * LF_M; i += LF_THREADS) sPSum[i] = 0.0f;

  int first_tile = lo / LF_KT, last_tile = hi / LF_KT;
  if (p.parts > 1) {                                         // this block's share of the key tiles (it may be empty)
    const int per = (last_tile - first_tile + p.parts) / p.parts;
    first_tile += static_cast<int>(blockIdx.z) * per;
    last_tile = min(last_tile, first_tile + per - 1);
  }
  if (BULK) {
    if (warp == 0) lf_load_keys_bulk(p, table, sK, RS, RW, first_tile * LF_KT, lo, hi, lane, &lf_bar[0]);
  } else {
    lf_load_keys(p, table, sK, RS, RW, first_tile * LF_KT, lo, hi, warp, lane);
    lf_commit();
  }

  // the four units whose output this thread holds: g, g + 8, 16 + g, 24 + g; their positions and validity
  int upos[4];
  bool uok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int u = (i >> 1) * 16 + (i & 1) * 8 + g;
    const int ur = u / p.HG, uh = u % p.HG;
    uok[i] = ur < rows && uh < heads;
    upos[i] = pos0 + ur;
  }
  float m_run[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, l_run[4] = {0.f, 0.f, 0.f, 0.f};
  float o[2][NT][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < NT; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[a][b][c] = 0.0f;
  const int mt = warp & 1, kq = warp >> 1;
  const float scale2 = p.scale * LF_LOG2E;
  const int ksteps = RWp / 16;

  for (int kt = first_tile; kt <= last_tile; ++kt) {
    bf16* stage = sK + static_cast<size_t>((kt - first_tile) & 1) * LF_KT * RS;
    if (BULK) {
      const int ti = kt - first_tile;
      const bool ok = mbar_wait(&lf_bar[ti & 1], (ti >> 1) & 1, p.status, LF_ERR_COPY, &lf_abort);
      if (!__syncthreads_and(ok)) return;                   // (uniform: all leave, nothing is written)
      if (kt < last_tile && warp == 0)
        lf_load_keys_bulk(p, table, sK + static_cast<size_t>((ti + 1) & 1) * LF_KT * RS, RS, RW, (kt + 1) * LF_KT, lo, hi, lane,
                          &lf_bar[(ti + 1) & 1]);
    } else {
      lf_wait<0>();
      __syncthreads();                                      // the tile is here; everyone is done with the one before
      if (kt < last_tile) {
        lf_load_keys(p, table, sK + static_cast<size_t>((kt - first_tile + 1) & 1) * LF_KT * RS, RS, RW, (kt + 1) * LF_KT, lo, hi,
                     warp, lane);
        lf_commit();
      }
    }
    // ---- scores of (units 16 mt .. +15) x (keys 16 kq .. +15) ------------------------------------------------
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    if (mt == 0 || two) {
      const bf16* qa = sQ + static_cast<size_t>(mt * 16 + (lane & 15)) * RS + (lane >> 4) * 8;
      const bf16* kb = stage + static_cast<size_t>(kq * 16 + (lane & 7) + ((lane >> 4) << 3)) * RS + ((lane >> 3) & 1) * 8;
#pragma unroll 4
      for (int ks = 0; ks < ksteps; ++ks) {
        uint32_t a[4], b[4];
        lf_ldmatrix_x4(a, qa + ks * 16);
        lf_ldmatrix_x4(b, kb + ks * 16);
        lf_mma(s[0], a, b[0], b[1]);
        lf_mma(s[1], a, b[2], b[3]);
      }
    }
    // mask, scale, the maxima of this warp's 16 keys per unit
    const int tk = kt * LF_KT + kq * 16 + q4 * 2;           // key of s[0][0]; s[n][j]: + 8 n + (j & 1); j >= 2: unit + 8
    float pm[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = mt * 2 + (j >> 1);
        const int t = tk + 8 * n + (j & 1), gap = upos[i] - t;
        const bool see = uok[i] && gap >= 0 && (p.window == 0 || gap < p.window);
        s[n][j] = see ? s[n][j] * scale2 : -INFINITY;
        pm[j >> 1] = fmaxf(pm[j >> 1], s[n][j]);
      }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      pm[e] = fmaxf(pm[e], __shfl_xor_sync(0xffffffffu, pm[e], 1));
      pm[e] = fmaxf(pm[e], __shfl_xor_sync(0xffffffffu, pm[e], 2));
      if (q4 == 0) sPMax[kq * LF_M + mt * 16 + e * 8 + g] = pm[e];
    }
    __syncthreads();
    // ---- every thread: the new maxima of its four units, and the sums of the tile before ------------------------
    float corr[4], m_use[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int u = (i >> 1) * 16 + (i & 1) * 8 + g;
      const float m_tile = fmaxf(fmaxf(sPMax[u], sPMax[LF_M + u]), fmaxf(sPMax[2 * LF_M + u], sPMax[3 * LF_M + u]));
      const float m_new = fmaxf(m_run[i], m_tile);
      corr[i] = m_new == -INFINITY ? 1.0f : lf_exp2(m_run[i] - m_new);
      m_use[i] = m_new == -INFINITY ? 0.0f : m_new;
      m_run[i] = m_new;
    }
    // ---- P of this warp's scores, rounded to bf16; the sums per unit -------------------------------------------------
    float ps[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const float p0 = lf_exp2(s[n][0] - m_use[mt * 2]), p1 = lf_exp2(s[n][1] - m_use[mt * 2]);
      const float p2 = lf_exp2(s[n][2] - m_use[mt * 2 + 1]), p3 = lf_exp2(s[n][3] - m_use[mt * 2 + 1]);
      ps[0] += p0 + p1;
      ps[1] += p2 + p3;
      const int col = kq * 16 + n * 8 + q4 * 2;
      *reinterpret_cast<uint32_t*>(sP + static_cast<size_t>(mt * 16 + g) * LF_PS + col) = lf_pack(p0, p1);
      *reinterpret_cast<uint32_t*>(sP + static_cast<size_t>(mt * 16 + 8 + g) * LF_PS + col) = lf_pack(p2, p3);
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      ps[e] += __shfl_xor_sync(0xffffffffu, ps[e], 1);
      ps[e] += __shfl_xor_sync(0xffffffffu, ps[e], 2);
      if (q4 == 0) sPSum[kq * LF_M + mt * 16 + e * 8 + g] = ps[e];
    }
    __syncthreads();
    // ---- O <- corr O + P V -----------------------------------------------------------------------------------------
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int u = (i >> 1) * 16 + (i & 1) * 8 + g;
      l_run[i] = l_run[i] * corr[i] + ((sPSum[u] + sPSum[LF_M + u]) + (sPSum[2 * LF_M + u] + sPSum[3 * LF_M + u]));
    }
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int b = 0; b < NT; ++b) {
        o[a][b][0] *= corr[a * 2]; o[a][b][1] *= corr[a * 2];
        o[a][b][2] *= corr[a * 2 + 1]; o[a][b][3] *= corr[a * 2 + 1];
      }
    const int col0 = warp * NT * 8;
    if (col0 < p.R) {
#pragma unroll
      for (int kk = 0; kk < LF_KT / 16; ++kk) {
        uint32_t a0[4], a1[4] = {0u, 0u, 0u, 0u};
        lf_ldmatrix_x4(a0, sP + static_cast<size_t>(lane & 15) * LF_PS + kk * 16 + (lane >> 4) * 8);
        if (two) lf_ldmatrix_x4(a1, sP + static_cast<size_t>(16 + (lane & 15)) * LF_PS + kk * 16 + (lane >> 4) * 8);
        const bf16* vb = stage + static_cast<size_t>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * RS + col0 + (lane >> 4) * 8;
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          if (col0 + np * 16 < p.R) {
            uint32_t b[4];
            lf_ldmatrix_x4_trans(b, vb + np * 16);
            lf_mma(o[0][2 * np], a0, b[0], b[1]);
            lf_mma(o[0][2 * np + 1], a0, b[2], b[3]);
            if (two) {
              lf_mma(o[1][2 * np], a1, b[0], b[1]);
              lf_mma(o[1][2 * np + 1], a1, b[2], b[3]);
            }
          }
        }
      }
    }
  }
  if (p.parts > 1) {
    // ---- a part: (max, sum, O) of every unit to scratch; the merge kernel finishes --------------------------------------
    if (BULK) {                                              // (a part without key tiles has its one load in flight)
      if (first_tile > last_tile) mbar_wait(&lf_bar[0], 0, p.status, LF_ERR_COPY, &lf_abort);
    } else {
      lf_wait<0>();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (!uok[i]) continue;
      const int u = (i >> 1) * 16 + (i & 1) * 8 + g;
      const int ur = u / p.HG, uh = u % p.HG;
      float* rec = p.scratch + ((static_cast<size_t>(row0 + ur) * p.H + h0 + uh) * p.parts + blockIdx.z) * (p.R + 2);
      if (warp == 0 && q4 == 0) {
        rec[0] = m_run[i];
        rec[1] = l_run[i];
      }
#pragma unroll
      for (int b = 0; b < NT; ++b) {
        const int col = (warp * NT + b) * 8 + q4 * 2;
        if (col < p.R) {
          const int a = i >> 1, j = (i & 1) * 2;
          *reinterpret_cast<float2*>(rec + 2 + col) = make_float2(o[a][b][j], o[a][b][j + 1]);
        }
      }
    }
    return;
  }
  // ---- the sink joins the denominator; O / denominator out ---------------------------------------------------------
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (!uok[i]) continue;
    const int u = (i >> 1) * 16 + (i & 1) * 8 + g;
    const int ur = u / p.HG, uh = u % p.HG;
    float keep = 1.0f, den = l_run[i];
    if (p.sink) {
      const float sk = p.sink[h0 + uh] * LF_LOG2E;
      const float m_all = fmaxf(m_run[i], sk);
      keep = lf_exp2(m_run[i] - m_all);
      den = l_run[i] * keep + lf_exp2(sk - m_all);
    }
    const float f = keep / den;
    bf16* orow = p.out + static_cast<size_t>(row0 + ur) * p.out_stride + static_cast<size_t>(h0 + uh) * p.R;
#pragma unroll
    for (int b = 0; b < NT; ++b) {
      const int col = (warp * NT + b) * 8 + q4 * 2;
      if (col < p.R) {
        const int a = i >> 1, j = (i & 1) * 2;
        *reinterpret_cast<uint32_t*>(orow + col) = lf_pack(o[a][b][j] * f, o[a][b][j + 1] * f);
      }
    }
  }
}

// One block per (row, head): the parts' (max, sum, O) merged in the order of the parts, the sink added to the
// denominator, the output written. A part without keys has max -inf and weighs nothing.
__global__ void latent_merge_kernel(const float* __restrict__ scratch, const float* __restrict__ sink, bf16* __restrict__ out,
                                    int out_stride, int H, int R, int parts) {
  const int row = blockIdx.x, head = blockIdx.y;
  const float* rec = scratch + (static_cast<size_t>(row) * H + head) * parts * (R + 2);
  pdl_wait();
  pdl_trigger();
  float m_all = sink ? sink[head] * LF_LOG2E : -INFINITY;
  for (int k = 0; k < parts; ++k) m_all = fmaxf(m_all, rec[static_cast<size_t>(k) * (R + 2)]);
  float den = sink ? lf_exp2(sink[head] * LF_LOG2E - m_all) : 0.0f;
  for (int k = 0; k < parts; ++k) {
    const float m = rec[static_cast<size_t>(k) * (R + 2)];
    if (m != -INFINITY) den += rec[static_cast<size_t>(k) * (R + 2) + 1] * lf_exp2(m - m_all);
  }
  bf16* orow = out + static_cast<size_t>(row) * out_stride + static_cast<size_t>(head) * R;
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < parts; ++k) {
      const float m = rec[static_cast<size_t>(k) * (R + 2)];
      if (m != -INFINITY) acc = fmaf(rec[static_cast<size_t>(k) * (R + 2) + 2 + d], lf_exp2(m - m_all), acc);
    }
    orow[d] = __float2bfloat16_rn(acc / den);
  }
}

}  // namespace dl

// Shared memory a launch needs, for the host to check against the device's limit.
static size_t lf_smem_bytes(int R, int r) {
  const int RS = ((R + r + 15) & ~15) + 8;
  return sizeof(dl::bf16) * (static_cast<size_t>(dl::LF_M + 2 * dl::LF_KT) * RS + dl::LF_M * dl::LF_PS) + sizeof(float) * 8 * dl::LF_M;
}

// qw: [rows, H * (R + r)] wide queries; cache: [pages, page_size, R + r]; tiles: n_tiles x (slot, first row, rows,
// first position), rows at most 32 / HG (HG = heads to a block: min(H, 32), or any divisor-free count up to 32);
// out: [rows, H * R]. R, r: multiples of 8, R at most 512. sink may be null. parts > 1: the keys of every tile are
// dealt over that many blocks, through scratch (float32 [rows, H, parts, R + 2]; `rows` rows are merged afterwards).
DL_EXPORT int dl_latent_attention_flash(const void* qw, int q_stride, const void* cache, const int* block_table, int max_blocks,
                                        const int* tiles, int n_tiles, const float* sink, void* out, int out_stride, int H, int R,
                                        int r, int page_size, float scale, int window, int HG, int parts, float* scratch,
                                        int rows, int bulk, int* status, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (bulk && status == nullptr) return DL_ERR_UNSUPPORTED;
  if (parts < 1 || parts > 64 || (parts > 1 && (scratch == nullptr || rows <= 0 || (reinterpret_cast<uintptr_t>(scratch) & 7) != 0)))
    return DL_ERR_UNSUPPORTED;
  if (H <= 0 || R <= 0 || R % 8 != 0 || r % 8 != 0 || r < 0 || R > 512 || page_size <= 0 || window < 0 || HG <= 0 || HG > 32 ||
      q_stride % 8 != 0 || out_stride % 2 != 0 || (reinterpret_cast<uintptr_t>(qw) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(cache) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 3) != 0 ||
      (reinterpret_cast<uintptr_t>(tiles) & 15) != 0)
    return DL_ERR_UNSUPPORTED;
  const size_t smem = lf_smem_bytes(R, r);
  if (smem > 220 * 1024) return DL_ERR_UNSUPPORTED;
  dl::LatentFlashParams p;
  p.qw = static_cast<const dl::bf16*>(qw);
  p.q_stride = q_stride;
  p.cache = static_cast<const dl::bf16*>(cache);
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.tiles = tiles;
  p.sink = sink;
  p.out = static_cast<dl::bf16*>(out);
  p.out_stride = out_stride;
  p.H = H; p.R = R; p.r = r; p.page_size = page_size; p.window = window; p.HG = HG;
  p.scale = scale;
  p.status = status;
  p.parts = parts;
  p.scratch = scratch;
  const int groups = (H + HG - 1) / HG;
  if (groups > 65535) return DL_ERR_UNSUPPORTED;
  dim3 grid(n_tiles, groups, parts);
  int code;
#define DL_LAUNCH2(NT, B)                                                                                                \
  do {                                                                                                                   \
    cudaError_t e = cudaFuncSetAttribute(dl::latent_attention_flash_kernel<NT, B>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         static_cast<int>(smem));                                                        \
    if (e != cudaSuccess) return static_cast<int>(e);                                                                    \
    code = dl::launch_streaming(dl::latent_attention_flash_kernel<NT, B>, grid, dim3(dl::LF_THREADS), smem, stream, p);   \
  } while (0)
#define DL_LAUNCH(NT)            \
  do {                           \
    if (bulk) DL_LAUNCH2(NT, true); \
    else DL_LAUNCH2(NT, false);  \
  } while (0)
  if (R <= 128) DL_LAUNCH(2);
  else if (R <= 256) DL_LAUNCH(4);
  else DL_LAUNCH(8);
#undef DL_LAUNCH
#undef DL_LAUNCH2
  if (code != 0 || parts == 1) return code;
  return dl::launch_streaming(dl::latent_merge_kernel, dim3(rows, H), dim3(128), 0, stream, static_cast<const float*>(scratch), sink,
                              static_cast<dl::bf16*>(out), out_stride, H, R, parts);
}
