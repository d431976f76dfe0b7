// One product a head on the tensor cores: y[m, b, :] = x[m, b, :] . w[b]^T for b < batches (the heads of a mixer
// whose heads each have a matrix of their own), bfloat16 operands, 32-bit sums, optionally times
// sigmoid(gate[m, b * N + n]) (32-bit gate) before the single rounding.  Tiles of 64 x 64 outputs a CTA of four
// warps (mma.sync m16n8k16: these products are small and many, K is a head's size or a latent's), operands
// staged through shared memory in blocks of 64 along K.  K must be a multiple of 8 and the operands 16-byte
// aligned; other shapes go to the plain kernel.
#include "common.cuh"

namespace lb {

constexpr int GH_BM = 64, GH_BN = 64, GH_BK = 64, GH_LD = GH_BK + 8;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__global__ void __launch_bounds__(128)
gemm_heads_mma_kernel(bf16* __restrict__ y, const bf16* __restrict__ x, const bf16* __restrict__ w, int M, int N, int K,
                      long long ldx, long long ldy, long long bx, long long bw, long long by,
                      const float* __restrict__ gate, long long ldg) {
  __shared__ __align__(16) bf16 As[GH_BM][GH_LD];
  __shared__ __align__(16) bf16 Bs[GH_BN][GH_LD];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int m0 = blockIdx.y * GH_BM, n0 = blockIdx.x * GH_BN, b = blockIdx.z;
  x += (size_t)b * bx; w += (size_t)b * bw; y += (size_t)b * by;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += GH_BK) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + it * 128;                 // 512 pieces of 8 values a tile
      const int r = idx >> 3, c = (idx & 7) * 8;
      uint4 va = make_uint4(0u, 0u, 0u, 0u), vb = va;
      if (k0 + c < K) {
        if (m0 + r < M) va = *reinterpret_cast<const uint4*>(x + (size_t)(m0 + r) * ldx + k0 + c);
        if (n0 + r < N) vb = *reinterpret_cast<const uint4*>(w + (size_t)(n0 + r) * K + k0 + c);
      }
      *reinterpret_cast<uint4*>(&As[r][c]) = va;
      *reinterpret_cast<uint4*>(&Bs[r][c]) = vb;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GH_BK; kk += 16) {
      uint32_t a[4];
      const bf16* ar = &As[warp * 16 + g][kk + 2 * t4];
      a[0] = *reinterpret_cast<const uint32_t*>(ar);
      a[1] = *reinterpret_cast<const uint32_t*>(ar + 8 * GH_LD);
      a[2] = *reinterpret_cast<const uint32_t*>(ar + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(ar + 8 * GH_LD + 8);
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
        uint32_t bb[2];
        const bf16* br = &Bs[nb * 8 + g][kk + 2 * t4];
        bb[0] = *reinterpret_cast<const uint32_t*>(br);
        bb[1] = *reinterpret_cast<const uint32_t*>(br + 8);
        mma_bf16_16816(acc[nb], a, bb);
      }
    }
    __syncthreads();
  }
  if (gate) gate += (size_t)b * N;
#pragma unroll
  for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = m0 + warp * 16 + g + 8 * half;
      if (m >= M) continue;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int n = n0 + nb * 8 + 2 * t4 + j;
        if (n >= N) continue;
        float v = acc[nb][2 * half + j];
        if (gate) v *= 1.f / (1.f + expf(-gate[(size_t)m * ldg + n]));
        y[(size_t)m * ldy + n] = __float2bfloat16_rn(v);
      }
    }
  }
}

}  // namespace lb

// 1 when lb_gemm_heads_mma takes these sizes and addresses
LB_EXPORT int lb_gemm_heads_mma_ok(const void* y, const void* x, const void* w, int K, long long ldx, long long bx, long long bw) {
  return K % 8 == 0 && ldx % 8 == 0 && bx % 8 == 0 && bw % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && y != nullptr;
}

LB_EXPORT int lb_gemm_heads_mma(void* y, const void* x, const void* w, int batches, int M, int N, int K, long long ldx,
                                long long ldy, long long bx, long long bw, long long by, const float* gate, long long ldg,
                                cudaStream_t stream) {
  LB_CHECK_ARG(M >= 0 && N > 0 && K > 0 && batches > 0 && batches <= 65535 && ldx >= K && ldy >= N,
               "gemm_heads_mma: bad sizes batches=%d M=%d N=%d K=%d", batches, M, N, K);
  LB_CHECK_ARG(lb_gemm_heads_mma_ok(y, x, w, K, ldx, bx, bw), "gemm_heads_mma: K, strides and addresses must be multiples of 8 values (16 bytes)");
  LB_CHECK_ARG(gate == nullptr || ldg >= (long long)batches * N, "gemm_heads_mma: the gate's rows are shorter than batches * N");
  LB_CHECK_ARG((M + lb::GH_BM - 1) / lb::GH_BM <= 65535, "gemm_heads_mma: too many rows (%d)", M);
  if (M == 0) return 0;
  dim3 grid((N + lb::GH_BN - 1) / lb::GH_BN, (M + lb::GH_BM - 1) / lb::GH_BM, batches);
  lb::launch(lb::gemm_heads_mma_kernel, grid, dim3(128), 0, stream, (lb::bf16*)y, (const lb::bf16*)x, (const lb::bf16*)w, M, N, K,
             ldx, ldy, bx, bw, by, gate, ldg);
  LB_CHECK_LAUNCH("gemm_heads_mma");
  return 0;
}
