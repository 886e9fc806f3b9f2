// Block-diagonal (per-head) matrix product on bf16 tensor cores (mma.sync m16n8k16, fp32 accumulation):
//
//   out[row, h * head_out + j] = sum_i in[row, h * head_in + i] * W[h][i][j]        (i < n_in, j < n_out)
//
// optionally times sigmoid(gate[row, h * gate_head + j]) (the product rounded to bf16 first, as when it is a tensor of
// its own). The two per-head products of latent attention are of this kind (latent_attention.cu has the plain kernel
// for float32 and odd sizes). Block = (64 rows, head, 64 columns), four warps of 16 rows each; the inputs' and W's
// slices of 32 along i are double-buffered with cp.async; W is stored [i][j], so its fragments come through
// ldmatrix.trans. Sizes are run-time multiples of 8. The sum over i runs in a fixed order for every output.
#include "common.cuh"

namespace dl {

constexpr int HT_BM = 64, HT_BN = 64, HT_BK = 32, HT_THREADS = 128;
constexpr int HT_AS = HT_BK + 8;     // row stride of the input tile in shared memory (bf16)
constexpr int HT_BS = HT_BN + 8;     // row stride of the W tile

__device__ __forceinline__ void ht_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ht_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ht_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ht_cp16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}

__global__ void __launch_bounds__(HT_THREADS)
head_linear_tc_kernel(const bf16* __restrict__ in, int in_stride, int head_in, int n_in, const bf16* __restrict__ W, int n_out,
                      bf16* __restrict__ out, int out_stride, int head_out, const bf16* __restrict__ gate, int gate_stride,
                      int gate_head, int rows) {
  __shared__ __align__(16) bf16 sA[2][HT_BM * HT_AS];
  __shared__ __align__(16) bf16 sB[2][HT_BK * HT_BS];
  const int row0 = blockIdx.x * HT_BM, h = blockIdx.y, col0 = blockIdx.z * HT_BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, q4 = lane & 3;
  const bf16* a_base = in + static_cast<size_t>(h) * head_in;
  const bf16* w_base = W + static_cast<size_t>(h) * n_in * n_out;
  pdl_wait();
  pdl_trigger();

  auto load = [&](int stage, int k0) {
    // inputs: 64 rows x 4 pieces of 8; W: 32 rows x 8 pieces of 8
    for (int i = tid; i < HT_BM * (HT_BK / 8); i += HT_THREADS) {
      const int r = i / (HT_BK / 8), c = (i % (HT_BK / 8)) * 8;
      const bool ok = row0 + r < rows && k0 + c < n_in;
      ht_cp16(&sA[stage][r * HT_AS + c], ok ? a_base + static_cast<size_t>(row0 + r) * in_stride + k0 + c : in, ok);
    }
    for (int i = tid; i < HT_BK * (HT_BN / 8); i += HT_THREADS) {
      const int r = i / (HT_BN / 8), c = (i % (HT_BN / 8)) * 8;
      const bool ok = k0 + r < n_in && col0 + c < n_out;
      ht_cp16(&sB[stage][r * HT_BS + c], ok ? w_base + static_cast<size_t>(k0 + r) * n_out + col0 + c : W, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  float acc[HT_BN / 8][4];
#pragma unroll
  for (int n = 0; n < HT_BN / 8; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[n][j] = 0.0f;
  const int steps = (n_in + HT_BK - 1) / HT_BK;
  load(0, 0);
  for (int s = 0; s < steps; ++s) {
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();                                          // the slice is here; everyone is done with the one before
    if (s + 1 < steps) load((s + 1) & 1, (s + 1) * HT_BK);
    const bf16* A = sA[s & 1];
    const bf16* B = sB[s & 1];
#pragma unroll
    for (int kk = 0; kk < HT_BK / 16; ++kk) {
      uint32_t a[4];
      ht_ldmatrix_x4(a, A + (warp * 16 + (lane & 15)) * HT_AS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < HT_BN / 16; ++np) {
        uint32_t b[4];
        ht_ldmatrix_x4_trans(b, B + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * HT_BS + np * 16 + (lane >> 4) * 8);
        ht_mma(acc[2 * np], a, b[0], b[1]);
        ht_mma(acc[2 * np + 1], a, b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = row0 + warp * 16 + half * 8 + g;
    if (row >= rows) continue;
    bf16* orow = out + static_cast<size_t>(row) * out_stride + static_cast<size_t>(h) * head_out;
    const bf16* grow = gate ? gate + static_cast<size_t>(row) * gate_stride + static_cast<size_t>(h) * gate_head : nullptr;
#pragma unroll
    for (int n = 0; n < HT_BN / 8; ++n) {
      const int col = col0 + n * 8 + q4 * 2;
      if (col >= n_out) continue;
      float v0 = acc[n][half * 2], v1 = acc[n][half * 2 + 1];
      if (grow) {
        v0 = __bfloat162float(__float2bfloat16_rn(v0)) / (1.0f + expf(-__bfloat162float(grow[col])));
        v1 = __bfloat162float(__float2bfloat16_rn(v1)) / (1.0f + expf(-__bfloat162float(grow[col + 1])));
      }
      __nv_bfloat162 pr = __floats2bfloat162_rn(v0, v1);
      *reinterpret_cast<__nv_bfloat162*>(orow + col) = pr;
    }
  }
}

}  // namespace dl

// in: rows of in_stride elements, head h's inputs at column h * head_in; W: [H, n_in, n_out] contiguous; out likewise
// with out_stride and head_out; gate (may be null) with gate_stride and gate_head. bfloat16; n_in, n_out, the strides
// and the heads' offsets multiples of 8 (the output's: of 2), the arrays 16-byte aligned.
DL_EXPORT int dl_head_linear_tc(const void* in, int in_stride, int head_in, int n_in, const void* W, int n_out, void* out,
                                int out_stride, int head_out, const void* gate, int gate_stride, int gate_head, int rows,
                                int H, cudaStream_t stream) {
  if (rows <= 0 || H <= 0 || n_out <= 0) return 0;
  if (n_in <= 0 || n_in % 8 != 0 || n_out % 8 != 0 || in_stride % 8 != 0 || head_in % 8 != 0 || out_stride % 2 != 0 ||
      head_out % 2 != 0 || H > 65535 || (reinterpret_cast<uintptr_t>(in) & 15) != 0 || (reinterpret_cast<uintptr_t>(W) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(out) & 3) != 0)
    return DL_ERR_UNSUPPORTED;
  dim3 grid((rows + dl::HT_BM - 1) / dl::HT_BM, H, (n_out + dl::HT_BN - 1) / dl::HT_BN);
  if (grid.z > 65535) return DL_ERR_UNSUPPORTED;
  return dl::launch(dl::head_linear_tc_kernel, grid, dim3(dl::HT_THREADS), 0, stream, static_cast<const dl::bf16*>(in), in_stride,
                    head_in, n_in, static_cast<const dl::bf16*>(W), n_out, static_cast<dl::bf16*>(out), out_stride, head_out,
                    static_cast<const dl::bf16*>(gate), gate_stride, gate_head, rows);
}
