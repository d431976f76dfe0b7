// A feed-forward of many small experts of which every token uses a few: the router's choice, the lists of tokens
// by expert, the experts' products over those lists, and the weighted sum.
//
//   route      s = sigmoid(z) for the router's logits z (32-bit).  The choice is made on c = s + correction: the
//              experts form `groups` equal groups of neighbours, a group is worth the sum of its two largest c, only
//              the experts of the `keep` best groups can be chosen, and of those the `top` with the largest c are.
//              Ties go to the lower index.  The weights are the chosen experts' s (without the correction), divided
//              by their sum + 1e-20, times `scale`.
//   dispatch   the (token, choice) pairs sorted by expert: offsets of the experts' runs, the pair at each place and
//              the place of each pair, and the list of row tiles (expert, first place) the products walk.  One CTA;
//              nothing comes back to the host, so a step's launches do not depend on the choices.
//   product    y[place, :] = act(x[row(place), :] . W[e]^T) for the places of expert e, W [experts, N, K].  With
//              `gated`, W[e] holds N/2 gate rows and then N/2 up rows and y has N/2 columns (the activations of
//              swiglu.cu).  row(place) is the pair's token for the first product (`gather`), the place itself for the second.
//   combine    out[t, :] = sum_k weight[t, k] * y[place(t, k), :] (+ an expert every token uses), k in the order
//              of the choice, in 32-bit.
//
// Every output element is one thread's sum over k in increasing order, so a token's result does not depend on where
// the token stands in its expert's list, nor on the batch.
#include "common.cuh"

namespace lb {

// ---- route -----------------------------------------------------------------------------------------------------
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

__global__ void route_topk_kernel(int* __restrict__ ids, float* __restrict__ weights, const float* __restrict__ logits,
                                  long long ld, const float* __restrict__ correction, int num_tokens, int experts, int top,
                                  int groups, int keep, float scale) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int t = blockIdx.x * nwarps + warp;
  if (t >= num_tokens) return;
  float* s = smem + (size_t)warp * 3 * experts;     // plain scores
  float* c = s + experts;                           // choice scores
  float* gw = c + experts;                          // what a group is worth; then the sum of the chosen scores
  const int size = experts / groups;
  for (int e = lane; e < experts; e += 32) {
    const float v = 1.f / (1.f + expf(-logits[(size_t)t * ld + e]));
    s[e] = v;
    c[e] = v + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (groups > 1) {
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;           // the two largest of the group
      for (int j = 0; j < size; ++j) {
        const float v = c[g * size + j];
        if (v > a) { b = a; a = v; } else if (v > b) b = v;
      }
      gw[g] = size > 1 ? a + b : a;
    }
    __syncwarp();
    // the `keep` best groups get +inf as their mark; then every expert outside them leaves the choice
    for (int r = 0; r < keep; ++r) {
      float bv = -INFINITY; int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = gw[g];
        if (v != INFINITY && (v > bv || (v == bv && g < bi))) { bv = v; bi = g; }
      }
      warp_argmax(bv, bi);
      if (lane == 0 && bi < groups) gw[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (gw[e / size] != INFINITY) c[e] = -INFINITY;
    __syncwarp();
  }
  float sum = 0.f;                                    // the same on every lane
  for (int r = 0; r < top; ++r) {
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = c[e];
      if (!isnan(v) && (v > bv || (v == bv && e < bi))) { bv = v; bi = e; }
    }
    warp_argmax(bv, bi);
    if (bi >= experts) bi = 0;                        // nothing left to choose from: cannot happen with top <= keep * size
    sum += s[bi];
    if (lane == 0) { ids[(size_t)t * top + r] = bi; c[bi] = NAN; }      // NaN marks a chosen expert (-inf is a legal score)
    __syncwarp();
  }
  const float f = scale / (sum + 1e-20f);
  for (int r = lane; r < top; r += 32) weights[(size_t)t * top + r] = s[ids[(size_t)t * top + r]] * f;
}

// ---- dispatch --------------------------------------------------------------------------------------------------
// meta: [0] number of row tiles, then (expert, first place, end place) per tile from meta[4] on.
__global__ void expert_dispatch_kernel(const int* __restrict__ ids, int pairs, int experts, int tile_rows, int* __restrict__ offsets,
                                       int* __restrict__ pair_at, int* __restrict__ place_of, int* __restrict__ meta) {
  extern __shared__ int ism[];
  pdl_trigger();
  pdl_wait();
  int* count = ism;                 // [experts]
  int* start = ism + experts;       // [experts + 1]
  int* tile0 = start + experts + 1; // [experts + 1]
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  // a pair's rank among its expert's pairs: whatever order the atomics give; the order never shows in a result
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) place_of[i] = atomicAdd(&count[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0, tl = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = a; tile0[e] = tl;
      a += count[e]; tl += (count[e] + tile_rows - 1) / tile_rows;
    }
    start[experts] = a; tile0[experts] = tl;
    meta[0] = tl;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = start[e];
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int place = start[ids[i]] + place_of[i];
    place_of[i] = place;
    pair_at[place] = i;
  }
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int n = tile0[e + 1] - tile0[e];
    for (int j = 0; j < n; ++j) {
      int* m = meta + 4 + 3 * (tile0[e] + j);
      m[0] = e; m[1] = start[e] + j * tile_rows; m[2] = min(start[e + 1], start[e] + (j + 1) * tile_rows);
    }
  }
}

// The same sort with every expert's run padded to whole tiles of `tile` places, for products that take their rows
// from a matrix by whole tiles (the tensor-memory product): place_of [pairs], pair_at [places] (-1 where a place is
// padding), tile_group [places / tile] (the expert of each tile; the tiles behind the last run name expert 0 and hold padding).
__global__ void expert_dispatch_padded_kernel(const int* __restrict__ ids, int pairs, int experts, int tile, int places,
                                              int* __restrict__ pair_at, int* __restrict__ place_of, int* __restrict__ tile_group) {
  extern __shared__ int ism[];
  pdl_trigger();
  pdl_wait();
  int* count = ism;                 // [experts]
  int* start = ism + experts;       // [experts + 1]
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  for (int i = threadIdx.x; i < places; i += blockDim.x) pair_at[i] = -1;
  for (int i = threadIdx.x; i < places / tile; i += blockDim.x) tile_group[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) place_of[i] = atomicAdd(&count[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0;
    for (int e = 0; e < experts; ++e) { start[e] = a; a += (count[e] + tile - 1) / tile * tile; }
    start[experts] = a;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int place = start[ids[i]] + place_of[i];
    place_of[i] = place;
    pair_at[place] = i;
  }
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    for (int t = start[e] / tile; t < start[e + 1] / tile; ++t) tile_group[t] = e;
}

// xs[place, :] = x[pair_at[place] / top, :] (zeros where the place is padding), 16 bytes a thread
__global__ void expert_gather_rows_kernel(uint4* __restrict__ xs, const uint4* __restrict__ x, const int* __restrict__ pair_at,
                                          int top, int row_words) {
  pdl_trigger();
  pdl_wait();
  const int place = blockIdx.x, pair = pair_at[place];
  uint4* dst = xs + (size_t)place * row_words;
  if (pair < 0) {
    for (int i = threadIdx.x; i < row_words; i += blockDim.x) dst[i] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const uint4* src = x + (size_t)(pair / top) * row_words;
  for (int i = threadIdx.x; i < row_words; i += blockDim.x) dst[i] = src[i];
}

// ---- product ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float expert_act(int act, float limit, float g, float u) {
  if (act == 1) return fmaxf(g, 0.f) * u;
  if (act == 2) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  if (act == 3) {
    g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + expf(-1.702f * g)) * (u + 1.f);
  }
  return g / (1.f + expf(-g)) * u;
}

constexpr int EX_BM = 64, EX_BN = 64, EX_BK = 16;

struct ExpertGemmParams {
  void* y; const void* x; const void* w;
  const int* meta; const int* pair_at;
  int N, K, top;            // N: rows of W[e] (2 * columns of y when gated)
  long long ldx, ldy;
  int gather;               // 1: x row of a place = pair_at[place] / top; 0: the place
  int gated, act; float limit;
  int interleaved;          // gated only: gate and up rows alternate in blocks of 64 (gate rows of 64 features, then their up rows)
};

// rows of W[e] that hold the gate and the up weights of output column n
__device__ __forceinline__ void gate_up_rows(const ExpertGemmParams& p, int n, int ncols, int& gate_row, int& up_row) {
  if (p.interleaved) { gate_row = (n >> 6) * 128 + (n & 63); up_row = gate_row + 64; }
  else { gate_row = n; up_row = ncols + n; }
}

// ordinary pipes, any types: a tile of 64 places x 64 output columns, k in increasing order by one thread an element
template <typename TX, typename TW, typename TY, bool GATED>
__global__ void __launch_bounds__(256) expert_gemm_plain_kernel(ExpertGemmParams p) {
  __shared__ float xs[EX_BK][EX_BM + 4];
  __shared__ float ws[GATED ? 2 : 1][EX_BK][EX_BN + 4];
  __shared__ int src_row[EX_BM];
  pdl_trigger();
  pdl_wait();
  if ((int)blockIdx.y >= p.meta[0]) return;
  const int* m = p.meta + 4 + 3 * blockIdx.y;
  const int e = m[0], r0 = m[1], r1 = m[2];
  const int tid = threadIdx.x;
  const int ncols = GATED ? p.N / 2 : p.N;              // output columns
  const int n0 = blockIdx.x * EX_BN;
  const TX* x = (const TX*)p.x;
  const TW* w = (const TW*)p.w + (size_t)e * p.N * p.K;
  if (tid < EX_BM) {
    const int place = r0 + tid;
    src_row[tid] = place < r1 ? (p.gather ? p.pair_at[place] / p.top : place) : -1;
  }
  __syncthreads();
  const int tr = tid / 16, tc = tid % 16;               // rows tr * 4 .., columns tc * 4 ..
  float acc[4][4], acc2[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; acc2[i][j] = 0.f; }
  for (int k0 = 0; k0 < p.K; k0 += EX_BK) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + it * 256;                   // 1024 = 64 rows x 16
      const int r = idx / EX_BK, c = idx % EX_BK;
      const int row = src_row[r], gk = k0 + c;
      xs[c][r] = (row >= 0 && gk < p.K) ? to_f32(x[(size_t)row * p.ldx + gk]) : 0.f;
    }
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + it * 256;                   // 1024 = 64 rows x 16
      const int r = idx / EX_BK, c = idx % EX_BK;
      const int gn = n0 + r, gk = k0 + c;
      const bool ok = gn < ncols && gk < p.K;
      int gr = gn, ur = gn;
      if (GATED) gate_up_rows(p, gn, ncols, gr, ur);
      ws[0][c][r] = ok ? to_f32(w[(size_t)gr * p.K + gk]) : 0.f;
      if (GATED) ws[1][c][r] = ok ? to_f32(w[(size_t)ur * p.K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < EX_BK; ++kk) {
      float a[4], b[4], b2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][tr * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) { b[j] = ws[0][kk][tc * 4 + j]; b2[j] = GATED ? ws[1][kk][tc * 4 + j] : 0.f; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (GATED) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
  TY* y = (TY*)p.y;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int place = r0 + tr * 4 + i;
    if (place >= r1) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tc * 4 + j;
      if (gn >= ncols) continue;
      const float v = GATED ? expert_act(p.act, p.limit, acc[i][j], acc2[i][j]) : acc[i][j];
      y[(size_t)place * p.ldy + gn] = from_f32<TY>(v);
    }
  }
}

// tensor cores (mma.sync m16n8k16), bfloat16 operands, 32-bit sums: a tile of 64 places x 128 output columns a CTA of
// eight warps (warp w: rows (w & 1) * 32 .., columns (w >> 1) * 32 ..); K in blocks of 32 through four stages of shared
// memory that 16-byte asynchronous copies fill three blocks ahead of the tensor cores (with a few tokens the kernel
// streams the experts' weights, and the copies in flight are what fills the memory pipe); fragments by ldmatrix from
// rows padded to 80 bytes.  K a multiple of 8, 16-byte aligned rows.
constexpr int EM_BM = 64, EM_BK = 32, EM_LD = EM_BK + 8, EM_STAGES = 4;

__device__ __forceinline__ void ex_mma_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void ex_ldmatrix_x4(const void* addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(addr)));
}
__device__ __forceinline__ void ex_cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;             // 0: the 16 bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(n) : "memory");
}

template <bool GATED, int BN>
constexpr int expert_mma_smem() { return EM_STAGES * (EM_BM + (GATED ? 2 : 1) * BN) * EM_LD * 2; }

// BN: output columns of a tile, 128 or 64 (with few places a launch is a stream of weights, and narrower tiles are more
// CTAs to share it out over the SMs)
template <typename TY, bool GATED, int BN>
__global__ void __launch_bounds__(256) expert_gemm_mma_kernel(ExpertGemmParams p) {
  constexpr int EM_BN = BN;
  constexpr int NW = BN / 32;                                     // blocks of 8 columns a warp: 4 or 2
  extern __shared__ __align__(16) uint8_t ex_smem[];
  constexpr int NB = GATED ? 2 : 1;
  bf16* As = reinterpret_cast<bf16*>(ex_smem);                    // [stage][BM][LD]
  bf16* Bs = As + EM_STAGES * EM_BM * EM_LD;                      // [stage][NB][BN][LD]
  __shared__ int src_row[EM_BM];
  pdl_trigger();
  pdl_wait();
  if ((int)blockIdx.y >= p.meta[0]) return;
  const int* m = p.meta + 4 + 3 * blockIdx.y;
  const int e = m[0], r0 = m[1], r1 = m[2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int wm = (warp & 1) * 32, wn = (warp >> 1) * (BN / 4);
  const int ncols = GATED ? p.N / 2 : p.N;
  const int n0 = blockIdx.x * EM_BN;
  const bf16* x = (const bf16*)p.x;
  const bf16* w = (const bf16*)p.w + (size_t)e * p.N * p.K;
  if (tid < EM_BM) {
    const int place = r0 + tid;
    src_row[tid] = place < r1 ? (p.gather ? p.pair_at[place] / p.top : place) : -1;
  }
  __syncthreads();
  const int a_r = tid >> 2, a_c = (tid & 3) * 8;                  // this thread's piece of A: 64 rows x 4 pieces
  const int a_row = src_row[a_r];
  auto load_stage = [&](int st, int k0) {
    ex_cp_async16(As + (st * EM_BM + a_r) * EM_LD + a_c, a_row >= 0 ? x + (size_t)a_row * p.ldx + k0 + a_c : x, a_row >= 0 && k0 + a_c < p.K);
#pragma unroll
    for (int it = 0; it < BN / 64; ++it) {
      const int idx = tid + it * 256, r = idx >> 2, c = (idx & 3) * 8;   // BN rows x 4 pieces
      const bool ok = n0 + r < ncols && k0 + c < p.K;
      int gr = n0 + r, ur = n0 + r;
      if (GATED) gate_up_rows(p, n0 + r, ncols, gr, ur);
      ex_cp_async16(Bs + ((st * NB + 0) * EM_BN + r) * EM_LD + c, ok ? w + (size_t)gr * p.K + k0 + c : w, ok);
      if (GATED) ex_cp_async16(Bs + ((st * NB + 1) * EM_BN + r) * EM_LD + c, ok ? w + (size_t)ur * p.K + k0 + c : w, ok);
    }
  };
  float acc[2][NW][4], acc2[GATED ? 2 : 1][NW][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < NW; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) { acc[i][j][k] = 0.f; if (GATED) acc2[i][j][k] = 0.f; }
  const int nk = (p.K + EM_BK - 1) / EM_BK;
#pragma unroll
  for (int st = 0; st < EM_STAGES - 1; ++st) {
    if (st < nk) load_stage(st, st * EM_BK);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  // ldmatrix addresses of this lane: A rows (lane & 7) + 8 * ((lane >> 3) & 1), k half (lane >> 4); B rows (lane & 7) + 8 * (lane >> 4),
  // k half (lane >> 3) & 1
  const int a_lr = (lane & 7) + ((lane >> 3) & 1) * 8, a_lk = (lane >> 4) * 8;
  const int b_lr = (lane & 7) + (lane >> 4) * 8, b_lk = ((lane >> 3) & 1) * 8;
  for (int kb = 0; kb < nk; ++kb) {
    const int st = kb % EM_STAGES;
    asm volatile("cp.async.wait_group %0;" ::"n"(EM_STAGES - 2) : "memory");   // block kb has landed
    __syncthreads();                                                           // and the stage of block kb - 1 is free
    if (kb + EM_STAGES - 1 < nk) load_stage((kb + EM_STAGES - 1) % EM_STAGES, (kb + EM_STAGES - 1) * EM_BK);
    asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
    for (int kk = 0; kk < EM_BK; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
        ex_ldmatrix_x4(As + (st * EM_BM + wm + mi * 16 + a_lr) * EM_LD + kk + a_lk, a[mi][0], a[mi][1], a[mi][2], a[mi][3]);
#pragma unroll
      for (int nb = 0; nb < NW; nb += 2) {
        uint32_t b0, b1, b2, b3;
        ex_ldmatrix_x4(Bs + ((st * NB + 0) * EM_BN + wn + nb * 8 + b_lr) * EM_LD + kk + b_lk, b0, b1, b2, b3);
        const uint32_t lo[2] = {b0, b1}, hi[2] = {b2, b3};
        ex_mma_16816(acc[0][nb], a[0], lo); ex_mma_16816(acc[1][nb], a[1], lo);
        ex_mma_16816(acc[0][nb + 1], a[0], hi); ex_mma_16816(acc[1][nb + 1], a[1], hi);
        if (GATED) {
          ex_ldmatrix_x4(Bs + ((st * NB + 1) * EM_BN + wn + nb * 8 + b_lr) * EM_LD + kk + b_lk, b0, b1, b2, b3);
          const uint32_t lo2[2] = {b0, b1}, hi2[2] = {b2, b3};
          ex_mma_16816(acc2[0][nb], a[0], lo2); ex_mma_16816(acc2[1][nb], a[1], lo2);
          ex_mma_16816(acc2[0][nb + 1], a[0], hi2); ex_mma_16816(acc2[1][nb + 1], a[1], hi2);
        }
      }
    }
  }
  TY* y = (TY*)p.y;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int nb = 0; nb < NW; ++nb)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int place = r0 + wm + mi * 16 + g + 8 * half;
        if (place >= r1) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int n = n0 + wn + nb * 8 + 2 * t4 + j;
          if (n >= ncols) continue;
          const float v = GATED ? expert_act(p.act, p.limit, acc[mi][nb][2 * half + j], acc2[mi][nb][2 * half + j]) : acc[mi][nb][2 * half + j];
          y[(size_t)place * p.ldy + n] = from_f32<TY>(v);
        }
      }
}

// ---- combine ---------------------------------------------------------------------------------------------------
template <typename TO, typename TA>
__global__ void expert_combine_kernel(TO* __restrict__ out, const float* __restrict__ y, const float* __restrict__ weights,
                                      const int* __restrict__ place_of, const TA* __restrict__ always, int top, int width) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int j = threadIdx.x; j < width; j += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(weights[(size_t)t * top + k], y[(size_t)place_of[(size_t)t * top + k] * width + j], acc);
    if (always) acc += to_f32(always[(size_t)t * width + j]);
    out[(size_t)t * width + j] = from_f32<TO>(acc);
  }
}

}  // namespace lb

// ids [T, top] int32, weights [T, top] float32 from logits [T, ld] float32 and correction [experts] float32 (may be null)
LB_EXPORT int lb_route_topk(int* ids, float* weights, const float* logits, long long ld, const float* correction,
                            int num_tokens, int experts, int top, int groups, int keep, float scale, cudaStream_t stream) {
  LB_CHECK_ARG(ids && weights && logits, "route_topk: null argument");
  LB_CHECK_ARG(num_tokens >= 0 && experts > 0 && experts <= 4096 && top > 0 && top <= experts && groups > 0 && experts % groups == 0 &&
               keep > 0 && keep <= groups && top <= keep * (experts / groups) && ld >= experts,
               "route_topk: bad sizes experts=%d top=%d groups=%d keep=%d", experts, top, groups, keep);
  if (num_tokens == 0) return 0;
  const int warps = experts > 1024 ? 1 : 4;
  const size_t smem = (size_t)warps * 3 * experts * sizeof(float);
  lb::launch(lb::route_topk_kernel, dim3((num_tokens + warps - 1) / warps), dim3(warps * 32), smem, stream, ids, weights, logits, ld,
             correction, num_tokens, experts, top, groups, keep, scale);
  LB_CHECK_LAUNCH("route_topk");
  return 0;
}

// The row tiles of the experts' products have this many places.
LB_EXPORT int lb_expert_tile_rows() { return lb::EX_BM; }

// ids [pairs] -> offsets [experts + 1], pair_at [pairs], place_of [pairs], meta [4 + 3 * (pairs / tile_rows + experts)]
LB_EXPORT int lb_expert_dispatch(const int* ids, int pairs, int experts, int* offsets, int* pair_at, int* place_of, int* meta,
                                 cudaStream_t stream) {
  LB_CHECK_ARG(ids && offsets && pair_at && place_of && meta, "expert_dispatch: null argument");
  LB_CHECK_ARG(pairs >= 0 && experts > 0 && experts <= 4096, "expert_dispatch: bad sizes pairs=%d experts=%d", pairs, experts);
  static_assert(lb::EX_BM == lb::EM_BM, "both products walk the same row tiles");
  const size_t smem = (size_t)(3 * experts + 2) * sizeof(int);
  lb::launch(lb::expert_dispatch_kernel, dim3(1), dim3(1024), smem, stream, ids, pairs, experts, (int)lb::EX_BM, offsets, pair_at, place_of, meta);
  LB_CHECK_LAUNCH("expert_dispatch");
  return 0;
}

// places: a multiple of tile, at least pairs + experts * (tile - 1) rounded up to it
LB_EXPORT int lb_expert_dispatch_padded(const int* ids, int pairs, int experts, int tile, int places, int* pair_at, int* place_of,
                                        int* tile_group, cudaStream_t stream) {
  LB_CHECK_ARG(ids && pair_at && place_of && tile_group, "expert_dispatch_padded: null argument");
  LB_CHECK_ARG(pairs >= 0 && experts > 0 && experts <= 4096 && tile > 0 && places % tile == 0 && places >= pairs + experts * (tile - 1),
               "expert_dispatch_padded: bad sizes pairs=%d experts=%d tile=%d places=%d", pairs, experts, tile, places);
  lb::launch(lb::expert_dispatch_padded_kernel, dim3(1), dim3(1024), (size_t)(2 * experts + 1) * sizeof(int), stream, ids, pairs, experts,
             tile, places, pair_at, place_of, tile_group);
  LB_CHECK_LAUNCH("expert_dispatch_padded");
  return 0;
}

// xs [places, width] = the rows of x [T, width] (2-byte elements, width a multiple of 8) that the places name
LB_EXPORT int lb_expert_gather_rows(void* xs, const void* x, const int* pair_at, int places, int top, int width, cudaStream_t stream) {
  LB_CHECK_ARG(xs && x && pair_at && places >= 0 && top > 0 && width > 0 && width % 8 == 0 && (uintptr_t)xs % 16 == 0 && (uintptr_t)x % 16 == 0,
               "expert_gather_rows: bad arguments");
  if (places == 0) return 0;
  lb::launch(lb::expert_gather_rows_kernel, dim3(places), dim3(128), 0, stream, (uint4*)xs, (const uint4*)x, pair_at, top, width / 8);
  LB_CHECK_LAUNCH("expert_gather_rows");
  return 0;
}

// y[place, :] = act(x[row(place)] . W[e]^T) over the row tiles of `meta`; max_tiles bounds their number (the grid).
// fast: 1 allows the tensor-core kernel (bfloat16 x and W, K a multiple of 8, 16-byte aligned rows).
LB_EXPORT int lb_expert_gemm(void* y, int y_dtype, const void* x, int x_dtype, const void* w, int w_dtype, const int* meta,
                             const int* pair_at, int max_tiles, int N, int K, long long ldx, long long ldy, int top, int gather,
                             int gated, int act, float limit, int fast, int interleaved, cudaStream_t stream) {
  LB_CHECK_ARG(!interleaved || (gated && N % 128 == 0), "expert_gemm: interleaved gate and up rows come in blocks of 64");
  LB_CHECK_ARG(lb::valid_dtype(y_dtype) && lb::valid_dtype(x_dtype) && lb::valid_dtype(w_dtype), "expert_gemm: bad dtype");
  LB_CHECK_ARG(y && x && w && meta && pair_at && N > 0 && K > 0 && top > 0 && max_tiles >= 0 && (!gated || N % 2 == 0) && ldx >= K,
               "expert_gemm: bad arguments N=%d K=%d", N, K);
  LB_CHECK_ARG(act >= 0 && act <= 3, "expert_gemm: unknown activation %d", act);
  LB_CHECK_ARG(max_tiles <= 65535, "expert_gemm: too many row tiles (%d)", max_tiles);
  if (max_tiles == 0) return 0;
  lb::ExpertGemmParams p;
  p.y = y; p.x = x; p.w = w; p.meta = meta; p.pair_at = pair_at; p.N = N; p.K = K; p.top = top; p.ldx = ldx; p.ldy = ldy;
  p.gather = gather; p.gated = gated; p.act = act; p.limit = limit; p.interleaved = interleaved;
  const int ncols = gated ? N / 2 : N;
  const bool mma = fast && x_dtype == LB_BF16 && w_dtype == LB_BF16 && K % 8 == 0 && ldx % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0;
  if (mma) {
    static bool attr_set = false;
    if (!attr_set) {       // the stages need more shared memory than a launch gets unasked
      cudaFuncSetAttribute(lb::expert_gemm_mma_kernel<float, true, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, lb::expert_mma_smem<true, 128>());
      cudaFuncSetAttribute(lb::expert_gemm_mma_kernel<lb::bf16, true, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, lb::expert_mma_smem<true, 128>());
      cudaFuncSetAttribute(lb::expert_gemm_mma_kernel<float, false, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, lb::expert_mma_smem<false, 128>());
      cudaFuncSetAttribute(lb::expert_gemm_mma_kernel<lb::bf16, false, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, lb::expert_mma_smem<false, 128>());
      cudaFuncSetAttribute(lb::expert_gemm_mma_kernel<float, true, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, lb::expert_mma_smem<true, 64>());
      cudaFuncSetAttribute(lb::expert_gemm_mma_kernel<lb::bf16, true, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, lb::expert_mma_smem<true, 64>());
      attr_set = true;
    }
    // few row tiles and a gated product (two weight rows a column): tiles of 64 columns, twice the CTAs for the same weights
    const bool narrow = gated && (long long)max_tiles * ((ncols + 127) / 128) < 2 * 148;
    if (narrow) {
      dim3 grid((ncols + 63) / 64, max_tiles);
      LB_DISPATCH_DTYPE(y_dtype, TY, {
        lb::launch(lb::expert_gemm_mma_kernel<TY, true, 64>, grid, dim3(256), lb::expert_mma_smem<true, 64>(), stream, p);
      })
    } else {
      dim3 grid((ncols + 127) / 128, max_tiles);
      LB_DISPATCH_DTYPE(y_dtype, TY, {
        if (gated) lb::launch(lb::expert_gemm_mma_kernel<TY, true, 128>, grid, dim3(256), lb::expert_mma_smem<true, 128>(), stream, p);
        else lb::launch(lb::expert_gemm_mma_kernel<TY, false, 128>, grid, dim3(256), lb::expert_mma_smem<false, 128>(), stream, p);
      })
    }
  } else {
    dim3 grid((ncols + lb::EX_BN - 1) / lb::EX_BN, max_tiles);
    LB_DISPATCH_DTYPE(x_dtype, TX, {
      LB_DISPATCH_DTYPE(w_dtype, TW, {
        LB_DISPATCH_DTYPE(y_dtype, TY, {
          if (gated) lb::launch(lb::expert_gemm_plain_kernel<TX, TW, TY, true>, grid, dim3(256), 0, stream, p);
          else lb::launch(lb::expert_gemm_plain_kernel<TX, TW, TY, false>, grid, dim3(256), 0, stream, p);
        })
      })
    })
  }
  LB_CHECK_LAUNCH("expert_gemm");
  return 0;
}

// out[t] = sum_k weights[t, k] * y[place_of[t, k]] (+ always[t]); y float32 [pairs, width]
LB_EXPORT int lb_expert_combine(void* out, int out_dtype, const float* y, const float* weights, const int* place_of,
                                const void* always, int always_dtype, int num_tokens, int top, int width, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && lb::valid_dtype(always_dtype) && out && y && weights && place_of && top > 0 && width > 0, "expert_combine: bad arguments");
  if (num_tokens <= 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  LB_DISPATCH_DTYPE(out_dtype, TO, {
    LB_DISPATCH_DTYPE(always_dtype, TA, {
      lb::launch(lb::expert_combine_kernel<TO, TA>, dim3(num_tokens), dim3(threads), 0, stream, (TO*)out, y, weights, place_of,
                 (const TA*)always, top, width);
    })
  })
  LB_CHECK_LAUNCH("expert_combine");
  return 0;
}
