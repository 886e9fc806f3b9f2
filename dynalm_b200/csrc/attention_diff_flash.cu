// Differential attention over a paged cache of per-token records on bf16 tensor cores (mma.sync m16n8k16),
// softmax, cap and the combination of the two maps in fp32. Two kernels from one body:
//
//   prompt portions   one block per (query tile of 64 rows of ONE request, head): each of the four warps owns 16
//                     query rows and walks all keys, 64 at a time, double-buffered with cp.async;
//   single tokens     one block per (row, KV head, chunk of 16 heads of its group, part of the keys): the query
//                     heads that share a KV head are the 16 rows of the tile, so keys and values are read once
//                     per KV head; each warp takes 16 of a tile's 64 keys, the warps' running (max, sum, acc) are
//                     merged through shared memory, and when a row's keys are dealt over several blocks each
//                     leaves its part in scratch for diff_merge_kernel to finish.
//
// Per head and map m (see attention_diff.cu for the layout of queries and records):
//   s = scale * q_m . k_m;  s <- cap * tanh(s / cap) (cap > 0);  a_m = softmax(s over keys t <= p) V
//   o = a_1 - lambda * a_2;  o <- o / sqrt(mean(o^2) + eps) * out_scale
// Key tiles begin at multiples of 64 in absolute position, so a row's arithmetic in the prompt kernel does not
// depend on where its portion was cut. P is rounded to bf16 for the P V product; everything else after the
// Q K^T product is fp32. Map size and value size are run-time multiples of 16 (map up to 128; values up to the
// template's bound), so one build serves every model.
#include "common.cuh"

namespace dl {

constexpr int DF_BN = 64;        // keys per tile
constexpr int DF_THREADS = 128;
constexpr int DF_TILE = 128;     // rows of a query tile as the host cuts them
constexpr int DF_BM = 64;        // query rows per block of the prompt kernel
constexpr float DF_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void df_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void df_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void df_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float df_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float df_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// c * tanh(x) = c - 2c / (1 + e^(2x)), with x2 = 2 x log2(e) and c2 = -2c given: absolute error of a few 1e-7 of c
// over the whole range, exact limits at both ends (e^(2x) = inf gives c, 0 gives -c). Four instructions, two of them on
// the special-function unit.
__device__ __forceinline__ float df_scaled_tanh(float x2, float c, float c2) {
  return fmaf(df_rcp(1.0f + df_exp2(x2)), c2, c);
}
__device__ __forceinline__ uint32_t df_pack(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ void df_cp16(uint32_t smem, const void* gmem, bool valid) {
  const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void df_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void df_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

struct DiffParams {
  const bf16* q;
  int q_stride;
  const bf16* cache;
  long long record;
  int k_off, v_off;
  const int* block_table;
  int max_blocks;
  bf16* out;
  int out_stride;
  int n_heads, n_kv_heads, dim, vd, page_shift;
  float scale, softcap;
  const float* lambda;
  float out_scale, eps;
};

// A part of a (row, head): per map (max in log2 units, sum, acc[vd]), 2 * (vd + 2) floats. Merges `n` parts that lie
// `stride` floats apart (n at most 32) into lane-held values: every lane ends with the merged (max, sum) of both maps and the
// acc of its own value columns d = lane, lane + 32, ...
template <int VDMAX>
__device__ __forceinline__ void df_merge_parts(const float* parts, int n, size_t stride, int vd, int lane, float (&mx)[2],
                                               float (&sum)[2], float (&acc)[2][VDMAX / 32 > 0 ? VDMAX / 32 : 1]) {
  constexpr int PL = VDMAX / 32 > 0 ? VDMAX / 32 : 1;
  // lane p holds part p's (max, sum) of both maps (n <= 32): the merged max and sum are two butterflies, and the
  // loads of the accumulators below depend on nothing but their addresses
  float w[2];
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    const float pm = lane < n ? parts[lane * stride + m * (vd + 2)] : -INFINITY;
    const float pl = lane < n ? parts[lane * stride + m * (vd + 2) + 1] : 0.0f;
    mx[m] = warp_max(pm);
    w[m] = pm == -INFINITY ? 0.0f : df_exp2(pm - mx[m]);
    sum[m] = warp_sum(pl * w[m]);
#pragma unroll
    for (int i = 0; i < PL; ++i) acc[m][i] = 0.0f;
  }
  for (int p = 0; p < n; ++p) {
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const float wp = __shfl_sync(0xffffffffu, w[m], p);
      const float* part = parts + p * stride + m * (vd + 2) + 2;
#pragma unroll
      for (int i = 0; i < PL; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) acc[m][i] = fmaf(part[d], wp, acc[m][i]);
      }
    }
  }
}

// The head's output from the merged maps, by one warp: difference, unit RMS over the values, scale; bf16 store.
template <int VDMAX>
__device__ __forceinline__ void df_finish_row(const float (&sum)[2], const float (&acc)[2][VDMAX / 32 > 0 ? VDMAX / 32 : 1], int vd,
                                              int lane, float lambda, float out_scale, float eps, bf16* orow) {
  constexpr int PL = VDMAX / 32 > 0 ? VDMAX / 32 : 1;
  const float inv1 = sum[0] > 0.0f ? 1.0f / sum[0] : 0.0f, inv2 = sum[1] > 0.0f ? 1.0f / sum[1] : 0.0f;
  float o[PL], ss = 0.0f;
#pragma unroll
  for (int i = 0; i < PL; ++i) {
    o[i] = lane + 32 * i < vd ? acc[0][i] * inv1 - lambda * (acc[1][i] * inv2) : 0.0f;
    ss = fmaf(o[i], o[i], ss);
  }
  ss = warp_sum(ss);
  const float mul = out_scale / sqrtf(ss / static_cast<float>(vd) + eps);
#pragma unroll
  for (int i = 0; i < PL; ++i)
    if (lane + 32 * i < vd) orow[lane + 32 * i] = __float2bfloat16_rn(o[i] * mul);
}

// tiles[i] = (request slot, first row of the step, rows, first position)   [prompt kernel]
// positions / row_slot per row                                            [single-token kernel]
template <int VDMAX, bool SINGLE, int MAPS>
__global__ void __launch_bounds__(DF_THREADS * (3 - MAPS), MAPS == 1 ? 2 : (VDMAX <= 64 ? 3 : 1))
diff_flash_kernel(DiffParams a, const int4* __restrict__ tiles, const int* __restrict__ positions,
                  const int* __restrict__ row_slot, float* __restrict__ scratch, int n_split) {
  constexpr int QROWS = SINGLE ? 16 : DF_BM;       // rows of the Q tile in shared memory
  constexpr int NKG = SINGLE ? 1 : DF_BN / 16;     // 16-key groups of a tile that one warp takes
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int dim = a.dim, vd = a.vd;
  const int LDQ = 2 * dim + 8, LDV = vd + 8;       // row strides in elements: 16 bytes of padding keep ldmatrix conflict-free
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
  bf16* Ks = Qs + QROWS * LDQ;                     // [2][DF_BN][LDQ]
  bf16* Vs = Ks + 2 * DF_BN * LDQ;                 // [2][DF_BN][LDV]

  // MAPS == 2: four warps, each with both maps of its 16 rows. MAPS == 1 (prompt portions only): eight warps, warps 0..3
  // take map 1 and warps 4..7 map 2 of the same four groups of 16 rows: half the accumulators a thread, so that twice as
  // many warps fit an SM and hide each other's latencies; the second map's output crosses shared memory at the end.
  constexpr int THREADS = DF_THREADS * (3 - MAPS);
  const int tid = threadIdx.x, lane = tid & 31, warp = (tid >> 5) & 3, my_map = MAPS == 1 ? tid >> 7 : 0;
  const int g = lane >> 2, t = lane & 3;
  const int group = a.n_heads / a.n_kv_heads;
  int req, row0, nrows, pos0, head0, kvh, nheads_here;
  if (SINGLE) {
    const int chunks = (group + 15) / 16;
    row0 = blockIdx.x;
    kvh = blockIdx.y / chunks;
    const int chunk = blockIdx.y % chunks;
    head0 = kvh * group + chunk * 16;
    nheads_here = min(16, group - chunk * 16);
    req = ck_request(row_slot[row0]);
    pos0 = positions[row0];
    nrows = 1;
  } else {
    // heads are the fast index of the grid: the host lists the tiles that read the most keys first, so the longest
    // blocks of all heads start first and the grid ends evenly
    constexpr int SUB = DF_TILE / DF_BM;
    const int4 tile = ck_tile(tiles[blockIdx.y / SUB]);
    const int sub = blockIdx.y % SUB;
    req = tile.x;
    row0 = tile.y + sub * DF_BM;
    nrows = min(DF_BM, tile.z - sub * DF_BM);
    pos0 = tile.w + sub * DF_BM;
    if (nrows <= 0) return;
    head0 = blockIdx.x;
    kvh = head0 / group;
    nheads_here = 1;
  }
  const int page_mask = (1 << a.page_shift) - 1;
  const int* table = a.block_table + static_cast<size_t>(req) * a.max_blocks;
  const int pos_last = pos0 + nrows - 1;
  int j_begin = 0, j_end = pos_last / DF_BN;       // key tiles j_begin .. j_end
  if (SINGLE && n_split > 1) {
    const int total = j_end + 1, per = (total + n_split - 1) / n_split;
    j_begin = blockIdx.z * per;
    j_end = min(total, j_begin + per) - 1;
  }

  // Q tile -> shared (rows past the end are zero): a row of the tile is a token (prompt) or a head (single token)
  const int CHQ = 2 * dim / 8;
  const uint32_t qs_base = static_cast<uint32_t>(__cvta_generic_to_shared(Qs));
  for (int c = tid; c < QROWS * CHQ; c += THREADS) {
    const int r = c / CHQ, ch = c % CHQ;
    const bool ok = SINGLE ? r < nheads_here : r < nrows;
    const int rr = ok ? r : 0;
    const bf16* src = SINGLE ? a.q + static_cast<size_t>(row0) * a.q_stride + static_cast<size_t>(head0 + rr) * 2 * dim + ch * 8
                             : a.q + static_cast<size_t>(row0 + rr) * a.q_stride + static_cast<size_t>(head0) * 2 * dim + ch * 8;
    df_cp16(qs_base + static_cast<uint32_t>((r * LDQ + ch * 8) * sizeof(bf16)), src, ok);
  }
  const uint32_t ks_base = static_cast<uint32_t>(__cvta_generic_to_shared(Ks));
  const uint32_t vs_base = static_cast<uint32_t>(__cvta_generic_to_shared(Vs));
  const int CHV = vd / 8;
  const size_t k_at = static_cast<size_t>(a.k_off) + static_cast<size_t>(kvh) * 2 * dim;
  const size_t v_at = static_cast<size_t>(a.v_off) + static_cast<size_t>(kvh) * vd;
  // Two threads (four in a block of eight warps) copy one key's record: its page is looked up once per tile and thread,
  // and the 16-byte pieces of the key's two maps and of its values go out without another dependent load in between.
  constexpr int TPK = THREADS / DF_BN;
  const int kv_r = tid / TPK, kv_half = tid % TPK;
  const uint32_t k_row = static_cast<uint32_t>(kv_r * LDQ * sizeof(bf16)), v_row = static_cast<uint32_t>(kv_r * LDV * sizeof(bf16));
  // the record of this thread's key of tile j (its number in the cache), -1 past the last key: looked up one
  // tile before its copies are issued, so that no copy waits for its page id
  auto find_record = [&](int j) -> int {
    const int key = j * DF_BN + kv_r;
    if (j > j_end || key > pos_last) return -1;
    return (ck_page(table, key >> a.page_shift, a.max_blocks) << a.page_shift) + (key & page_mask);
  };
  auto load_kv = [&](int slot, int stage) {
    const long long rec = static_cast<long long>(slot) * a.record;
    const uint32_t k_stage = ks_base + static_cast<uint32_t>(stage * DF_BN * LDQ * sizeof(bf16)) + k_row;
    const uint32_t v_stage = vs_base + static_cast<uint32_t>(stage * DF_BN * LDV * sizeof(bf16)) + v_row;
    const bool ok = slot >= 0;
    const bf16* ksrc = a.cache + (ok ? rec : 0) + k_at;
    const bf16* vsrc = a.cache + (ok ? rec : 0) + v_at;
    for (int ch = kv_half; ch < CHQ; ch += TPK) df_cp16(k_stage + ch * 16, ksrc + ch * 8, ok);
    for (int ch = kv_half; ch < CHV; ch += TPK) df_cp16(v_stage + ch * 16, vsrc + ch * 8, ok);
  };
  if (j_begin <= j_end) load_kv(find_record(j_begin), 0);
  df_commit();
  int rec_next = find_record(j_begin + 1);

  float o[MAPS][VDMAX / 8][4];
#pragma unroll
  for (int m = 0; m < MAPS; ++m)
#pragma unroll
    for (int i = 0; i < VDMAX / 8; ++i) { o[m][i][0] = o[m][i][1] = o[m][i][2] = o[m][i][3] = 0.0f; }
  float m_run[MAPS][2], l_run[MAPS][2];
#pragma unroll
  for (int m = 0; m < MAPS; ++m) { m_run[m][0] = m_run[m][1] = -INFINITY; l_run[m][0] = l_run[m][1] = 0.0f; }
  // position of the lane's two rows (a single token: all rows are the one position)
  const int pos_a = SINGLE ? pos0 : pos0 + warp * 16 + g, pos_b = SINGLE ? pos0 : pos_a + 8;
  const int q_row = (SINGLE ? 0 : warp * 16) + (lane & 7) + ((lane >> 3) & 1) * 8;
  const int kg0 = SINGLE ? warp : 0;               // first 16-key group of a tile that this warp takes
  const float cap = a.softcap;
  // raw score -> 2 log2(e) times the tanh argument (capped), or -> log2 units (not capped); the capped score in log2 units
  // is post * tanh
  const float pre = cap > 0.0f ? a.scale / cap * (2.0f * DF_LOG2E) : a.scale * DF_LOG2E;
  const float post = cap * DF_LOG2E, post2 = -2.0f * post;
  const int KS = dim / 16;

  for (int j = j_begin; j <= j_end; ++j) {
    const int stage = (j - j_begin) & 1;
    if (j < j_end) {
      load_kv(rec_next, stage ^ 1);
      rec_next = find_record(j + 2);
    }
    df_commit();
    df_wait<1>();
    __syncthreads();
    const bf16* kt = Ks + stage * DF_BN * LDQ;
    const bf16* vt = Vs + stage * DF_BN * LDV;
    const int key0 = j * DF_BN + kg0 * 16;
    const bool edge = key0 + NKG * 16 - 1 > (SINGLE ? pos0 : pos0 + warp * 16);
    uint32_t pf[MAPS][NKG][4];       // the maps' weights as bf16 A fragments
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
      const int q_map = MAPS == 2 ? m : my_map;       // which map's slice of queries and keys
      float s[NKG * 2][4];
#pragma unroll
      for (int i = 0; i < NKG * 2; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t qf[4];
        df_ldmatrix_x4(qf, Qs + q_row * LDQ + q_map * dim + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < NKG; ++np) {
          uint32_t kb[4];
          const int key = (kg0 + np) * 16 + (lane & 7) + (lane >> 4) * 8;
          df_ldmatrix_x4(kb, kt + key * LDQ + q_map * dim + ks * 16 + ((lane >> 3) & 1) * 8);
          df_mma(s[2 * np], qf, kb[0], kb[1]);
          df_mma(s[2 * np + 1], qf, kb[2], kb[3]);
        }
      }
      // scores in log2 units (capped when asked for), masked by position; online softmax; P as bf16 A fragments
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < NKG * 2; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[i][e] * pre;
          if (cap > 0.0f) v = df_scaled_tanh(v, post, post2);
          if (edge) {
            const int key = key0 + i * 8 + 2 * t + (e & 1);
            if (key > ((e >> 1) ? pos_b : pos_a)) v = -INFINITY;
          }
          s[i][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2], neg_m[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_run[m][h], mx[h]);
        // a row with no visible key so far (rows past the end of the tile) keeps max = -inf; its weights are zeros
        corr[h] = m_new == -INFINITY ? 1.0f : df_exp2(m_run[m][h] - m_new);
        m_run[m][h] = m_new;
        neg_m[h] = m_new == -INFINITY ? 0.0f : -m_new;
      }
      float ls[2] = {0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < NKG * 2; ++i) {
        const float p0 = df_exp2(s[i][0] + neg_m[0]), p1 = df_exp2(s[i][1] + neg_m[0]);
        const float p2 = df_exp2(s[i][2] + neg_m[1]), p3 = df_exp2(s[i][3] + neg_m[1]);
        ls[0] += p0 + p1;
        ls[1] += p2 + p3;
        pf[m][i >> 1][(i & 1) * 2] = df_pack(p0, p1);
        pf[m][i >> 1][(i & 1) * 2 + 1] = df_pack(p2, p3);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        ls[h] += __shfl_xor_sync(0xffffffffu, ls[h], 1);
        ls[h] += __shfl_xor_sync(0xffffffffu, ls[h], 2);
        l_run[m][h] = l_run[m][h] * corr[h] + ls[h];
      }
      if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
        for (int i = 0; i < VDMAX / 8; ++i) {
          o[m][i][0] *= corr[0]; o[m][i][1] *= corr[0];
          o[m][i][2] *= corr[1]; o[m][i][3] *= corr[1];
        }
      }
    }
    // O_m += P_m V for both maps: a value fragment is loaded once and serves both
#pragma unroll
    for (int kk = 0; kk < NKG; ++kk) {
#pragma unroll
      for (int dp = 0; dp < VDMAX / 16; ++dp) {
        if (dp * 16 < vd) {
          uint32_t vb[4];
          const int key = (kg0 + kk) * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          df_ldmatrix_x4_trans(vb, vt + key * LDV + dp * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int m = 0; m < MAPS; ++m) {
            df_mma(o[m][2 * dp], pf[m][kk], vb[0], vb[1]);
            df_mma(o[m][2 * dp + 1], pf[m][kk], vb[2], vb[3]);
          }
        }
      }
    }
    __syncthreads();     // every warp is done with this stage before the next prefetch overwrites it
  }
  df_wait<0>();

  const float lambda = a.lambda[0];
  if constexpr (!SINGLE) {
    // a row's values lie in the four lanes of its quad: difference, sum of squares over the quad, scale, store
    float inv[MAPS][2];
#pragma unroll
    for (int m = 0; m < MAPS; ++m)
#pragma unroll
      for (int h = 0; h < 2; ++h) inv[m][h] = l_run[m][h] > 0.0f ? 1.0f / l_run[m][h] : 0.0f;
    float* second = reinterpret_cast<float*>(Ks);     // [DF_BM][vd]: the second map's output on its way to the first map's warps
    if (MAPS == 1) {
      __syncthreads();                                // nobody reads the key tiles any more (and no copy is in flight)
      if (my_map == 1) {
#pragma unroll
        for (int i = 0; i < VDMAX / 8; ++i) {
          if (i * 8 < vd) {
            float* dst = second + (warp * 16 + g) * vd + i * 8 + 2 * t;
            *reinterpret_cast<float2*>(dst) = make_float2(o[0][i][0] * inv[0][0], o[0][i][1] * inv[0][0]);
            *reinterpret_cast<float2*>(dst + 8 * vd) = make_float2(o[0][i][2] * inv[0][1], o[0][i][3] * inv[0][1]);
          }
        }
      }
      __syncthreads();
      if (my_map == 1) return;
    }
    float ss[2] = {0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < VDMAX / 8; ++i) {
      if (i * 8 < vd) {
        float other[4];
        if (MAPS == 1) {
          const float* src = second + (warp * 16 + g) * vd + i * 8 + 2 * t;
          const float2 lo = *reinterpret_cast<const float2*>(src), hi = *reinterpret_cast<const float2*>(src + 8 * vd);
          other[0] = lo.x; other[1] = lo.y; other[2] = hi.x; other[3] = hi.y;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          const float a2 = MAPS == 1 ? other[e] : o[MAPS - 1][i][e] * inv[MAPS - 1][h];
          const float v = o[0][i][e] * inv[0][h] - lambda * a2;
          o[0][i][e] = v;
          ss[h] = fmaf(v, v, ss[h]);
        }
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 1);
      ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 2);
      ss[h] = a.out_scale / sqrtf(ss[h] / static_cast<float>(vd) + a.eps);
    }
    const int r_a = warp * 16 + g, r_b = r_a + 8;
#pragma unroll
    for (int i = 0; i < VDMAX / 8; ++i) {
      if (i * 8 < vd) {
        const int col = head0 * vd + i * 8 + 2 * t;
        if (r_a < nrows)
          *reinterpret_cast<uint32_t*>(a.out + static_cast<size_t>(row0 + r_a) * a.out_stride + col) =
              df_pack(o[0][i][0] * ss[0], o[0][i][1] * ss[0]);
        if (r_b < nrows)
          *reinterpret_cast<uint32_t*>(a.out + static_cast<size_t>(row0 + r_b) * a.out_stride + col) =
              df_pack(o[0][i][2] * ss[1], o[0][i][3] * ss[1]);
      }
    }
    return;
  } else {
  // Single token: every warp leaves its part [16 rows][2 maps][(max, sum, acc[vd])] in shared memory (over the key
  // and value tiles, which nobody reads any more), then warp w merges the four parts of rows w, w + 4, ...
  float* parts = reinterpret_cast<float*>(smem_raw);
  const int row_floats = 2 * (vd + 2);
  const size_t warp_stride = static_cast<size_t>(16) * row_floats;
  __syncthreads();
#pragma unroll
  for (int m = 0; m < 2; ++m) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float* part = parts + warp * warp_stride + (g + 8 * h) * row_floats + m * (vd + 2);
      if (t == 0) {
        part[0] = m_run[m][h];
        part[1] = l_run[m][h];
      }
#pragma unroll
      for (int i = 0; i < VDMAX / 8; ++i) {
        if (i * 8 < vd) {
          part[2 + i * 8 + 2 * t] = o[m][i][2 * h];
          part[2 + i * 8 + 2 * t + 1] = o[m][i][2 * h + 1];
        }
      }
    }
  }
  __syncthreads();
  for (int r = warp; r < nheads_here; r += DF_THREADS / 32) {
    float mx[2], sum[2], acc[2][VDMAX / 32 > 0 ? VDMAX / 32 : 1];
    df_merge_parts<VDMAX>(parts + r * row_floats, DF_THREADS / 32, warp_stride, vd, lane, mx, sum, acc);
    const int head = head0 + r;
    if (n_split <= 1) {
      df_finish_row<VDMAX>(sum, acc, vd, lane, lambda, a.out_scale, a.eps,
                           a.out + static_cast<size_t>(row0) * a.out_stride + static_cast<size_t>(head) * vd);
    } else {
      float* dst = scratch + ((static_cast<size_t>(row0) * a.n_heads + head) * n_split + blockIdx.z) * row_floats;
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        if (lane == 0) {
          dst[m * (vd + 2)] = mx[m];
          dst[m * (vd + 2) + 1] = sum[m];
        }
#pragma unroll
        for (int i = 0; i < (VDMAX / 32 > 0 ? VDMAX / 32 : 1); ++i)
          if (lane + 32 * i < vd) dst[m * (vd + 2) + 2 + lane + 32 * i] = acc[m][i];
      }
    }
  }
  }
}

// Finishes the rows whose keys were dealt over n_split blocks: one warp per (row, head).
template <int VDMAX>
__global__ void __launch_bounds__(DF_THREADS)
diff_merge_kernel(const float* __restrict__ scratch, int n_split, int rows, int n_heads, int vd, const float* __restrict__ lambda,
                  float out_scale, float eps, bf16* __restrict__ out, int out_stride) {
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y * (DF_THREADS / 32) + (threadIdx.x >> 5);
  const int row = blockIdx.x;
  if (head >= n_heads) return;
  const int row_floats = 2 * (vd + 2);
  float mx[2], sum[2], acc[2][VDMAX / 32 > 0 ? VDMAX / 32 : 1];
  df_merge_parts<VDMAX>(scratch + (static_cast<size_t>(row) * n_heads + head) * n_split * row_floats, n_split, row_floats, vd, lane,
                        mx, sum, acc);
  df_finish_row<VDMAX>(sum, acc, vd, lane, lambda[0], out_scale, eps,
                       out + static_cast<size_t>(row) * out_stride + static_cast<size_t>(head) * vd);
}

inline size_t df_smem_bytes(bool single, int dim, int vd) {
  const size_t tiles = (static_cast<size_t>(single ? 16 : DF_BM) + 2 * DF_BN) * (2 * dim + 8) * sizeof(bf16) +
                       static_cast<size_t>(2) * DF_BN * (vd + 8) * sizeof(bf16);
  const size_t merge = single ? static_cast<size_t>(DF_THREADS / 32) * 16 * 2 * (vd + 2) * sizeof(float) : 0;
  return tiles > merge ? tiles : merge;
}

template <int VDMAX, bool SINGLE, int MAPS>
int df_launch(const DiffParams& a, dim3 grid, const int* tiles, const int* positions, const int* row_slot, float* scratch,
              int n_split, cudaStream_t stream) {
  const size_t smem = df_smem_bytes(SINGLE, a.dim, a.vd);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(diff_flash_kernel<VDMAX, SINGLE, MAPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = smem;
  }
  diff_flash_kernel<VDMAX, SINGLE, MAPS><<<grid, DF_THREADS * (3 - MAPS), smem, stream>>>(a, reinterpret_cast<const int4*>(tiles), positions,
                                                                      row_slot, scratch, n_split);
  return launch_status();
}

inline bool df_params(DiffParams& a, const void* q, int q_stride, const void* cache, long long record, int k_off, int v_off,
                      const int* block_table, int max_blocks, void* out, int out_stride, int n_heads, int n_kv_heads, int dim,
                      int vdim, int page_size, float scale, float softcap, const float* lambda, float out_scale, float eps) {
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  if ((1 << page_shift) != page_size || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads > 65535 || dim % 16 != 0 ||
      dim <= 0 || dim > 128 || vdim % 16 != 0 || vdim <= 0 || vdim > 128 || (q_stride & 7) || (out_stride & 1) ||
      (record & 7) || (k_off & 7) || (v_off & 7) || (reinterpret_cast<uintptr_t>(q) & 15) ||
      (reinterpret_cast<uintptr_t>(cache) & 15) || (reinterpret_cast<uintptr_t>(out) & 3) || !(scale > 0.0f) || softcap < 0.0f)
    return false;
  a = DiffParams{static_cast<const bf16*>(q), q_stride, static_cast<const bf16*>(cache), record, k_off, v_off, block_table,
                 max_blocks, static_cast<bf16*>(out), out_stride, n_heads, n_kv_heads, dim, vdim, page_shift, scale, softcap,
                 lambda, out_scale, eps};
  return true;
}

}  // namespace dl

// Prompt portions. bfloat16. tiles: int32 [n_tiles, 4] = (request slot, first row, rows <= 128, first position), 16-byte
// aligned. dim and vdim multiples of 16 up to 128; record, k_off, v_off multiples of 8 elements.
DL_EXPORT int dl_diff_attention_prefill(const void* q, int q_stride, const void* cache, long long record, int k_off, int v_off,
                                        const int* block_table, int max_blocks, const int* tiles, int n_tiles, void* out,
                                        int out_stride, int n_heads, int n_kv_heads, int dim, int vdim, int page_size,
                                        float scale, float softcap, const float* lambda, float out_scale, float eps,
                                        cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  dl::DiffParams a;
  if (!dl::df_params(a, q, q_stride, cache, record, k_off, v_off, block_table, max_blocks, out, out_stride, n_heads, n_kv_heads,
                     dim, vdim, page_size, scale, softcap, lambda, out_scale, eps))
    return DL_ERR_UNSUPPORTED;
  dim3 grid(n_heads, n_tiles * (dl::DF_TILE / dl::DF_BM));
  if (grid.y > 65535) return DL_ERR_UNSUPPORTED;
  // The maps are dealt over two sets of warps (half the registers a thread, twice the warps an SM): measured on B200 at
  // 2,048 tokens, us a layer, both maps in one warp / dealt: 16 heads of 64 + 64 with values of 128: 169 / 147; values of
  // 64: 148 / 124; maps and values of 128: 288 / 242; 32 heads of 32 with values of 64: 194 / 189.
  // DYNALM_DIFF_SPLIT_MAPS=0 keeps both maps in one warp (for measurements).
  static int forced = -2;
  if (forced == -2) { const char* e = getenv("DYNALM_DIFF_SPLIT_MAPS"); forced = e ? atoi(e) : -1; }
  const bool split_maps = forced != 0;
  if (vdim <= 32) return split_maps ? dl::df_launch<32, false, 1>(a, grid, tiles, nullptr, nullptr, nullptr, 1, stream)
                                    : dl::df_launch<32, false, 2>(a, grid, tiles, nullptr, nullptr, nullptr, 1, stream);
  if (vdim <= 64) return split_maps ? dl::df_launch<64, false, 1>(a, grid, tiles, nullptr, nullptr, nullptr, 1, stream)
                                    : dl::df_launch<64, false, 2>(a, grid, tiles, nullptr, nullptr, nullptr, 1, stream);
  return split_maps ? dl::df_launch<128, false, 1>(a, grid, tiles, nullptr, nullptr, nullptr, 1, stream)
                    : dl::df_launch<128, false, 2>(a, grid, tiles, nullptr, nullptr, nullptr, 1, stream);
}

// Rows that bring one token each (rows 0 .. rows - 1 of q and out). n_split > 1 deals every row's keys over that
// many blocks (at most 32); scratch then needs rows * n_heads * n_split * 2 * (vdim + 2) floats.
DL_EXPORT int dl_diff_attention_decode(const void* q, int q_stride, const void* cache, long long record, int k_off, int v_off,
                                       const int* block_table, int max_blocks, const int* positions, const int* row_slot,
                                       void* out, int out_stride, float* scratch, int rows, int n_heads, int n_kv_heads,
                                       int dim, int vdim, int page_size, float scale, float softcap, const float* lambda,
                                       float out_scale, float eps, int n_split, cudaStream_t stream) {
  if (rows <= 0) return 0;
  dl::DiffParams a;
  if (!dl::df_params(a, q, q_stride, cache, record, k_off, v_off, block_table, max_blocks, out, out_stride, n_heads, n_kv_heads,
                     dim, vdim, page_size, scale, softcap, lambda, out_scale, eps) || n_split < 1 || n_split > 32 ||
      (n_split > 1 && scratch == nullptr))
    return DL_ERR_UNSUPPORTED;
  const int group = n_heads / n_kv_heads;
  dim3 grid(rows, n_kv_heads * ((group + 15) / 16), n_split);
  if (grid.y > 65535) return DL_ERR_UNSUPPORTED;
  int rc;
  if (vdim <= 32) rc = dl::df_launch<32, true, 2>(a, grid, nullptr, positions, row_slot, scratch, n_split, stream);
  else if (vdim <= 64) rc = dl::df_launch<64, true, 2>(a, grid, nullptr, positions, row_slot, scratch, n_split, stream);
  else rc = dl::df_launch<128, true, 2>(a, grid, nullptr, positions, row_slot, scratch, n_split, stream);
  if (rc != 0 || n_split == 1) return rc;
  dim3 mgrid(rows, (n_heads + dl::DF_THREADS / 32 - 1) / (dl::DF_THREADS / 32));
#define DL_MERGE(V)                                                                                                     \
  dl::diff_merge_kernel<V><<<mgrid, dl::DF_THREADS, 0, stream>>>(scratch, n_split, rows, n_heads, vdim, lambda, out_scale, eps, \
                                                                 static_cast<dl::bf16*>(out), out_stride)
  if (vdim <= 32) DL_MERGE(32);
  else if (vdim <= 64) DL_MERGE(64);
  else DL_MERGE(128);
#undef DL_MERGE
  return dl::launch_status();
}
