// Gated linear recurrence with a lower-bounded forget gate that also sets what is written (HGRN2):
// per sequence and head, with a state S [dim, vdim] in 32-bit,
//
//   q_t = silu(a_t)                      a, b, v: this token's columns of the stacked input projection
//   f_t = l + (1 - l) * sigmoid(b_t + bias)
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T
//   o_t = S_t^T q_t
//
// for the tokens of a step, which are portions of several sequences; a sequence's state is read from its
// slot before its first token of the step and written back after its last.  Everything here is 32-bit.
//
// One CTA takes (32 value columns, one head, one sequence).  Its computing warps keep the state in registers:
// warp w rows w*DS .. w*DS+DS-1, one value column a lane, and walk the tokens in order.  Eight more warps
// feed them, a chunk of tokens at a time (16 tokens for heads of up to 128 rows, fewer for larger ones: 2048
// gate values a chunk, eight a feeding thread).  While the computing warps work on chunk c, the feeding warps
// turn the inputs of chunk c + 1, which they requested an iteration earlier, into gates in shared memory (two
// buffers), request the inputs of chunk c + 2, and add up, in warp order, the shares of o_t that the computing
// warps left for chunk c - 1; one barrier a chunk.  The order of every sum is fixed by (dim, DS) alone, so a
// token's result does not depend on how the sequence was cut into steps.
#include "common.cuh"

namespace lb {

constexpr int GR_FEED = 8;                      // feeding warps
constexpr int GR_FT = GR_FEED * 32;             // feeding threads
constexpr int GR_PER = 8;                       // gate values a feeding thread makes a chunk
constexpr int GR_TC_MAX = 16;                   // most tokens a chunk

struct GatedRecurrenceParams {
  const float* pre; long long ld;       // [T, ld]: q pre-activations at q_col, gate at f_col, values at v_col
  int q_col, f_col, v_col;
  const float* bias; const float* lower;   // [heads * dim]
  float* state;                         // [slots + 1, heads, dim, vdim]
  float* out;                           // [T, heads * vdim]
  const int* cu_tokens; const int* slots;
  int heads, dim, vdim;
};

__host__ __device__ inline int gr_chunk_tokens(int dimp) {
  int tc = GR_FT * GR_PER / dimp;
  return tc > GR_TC_MAX ? GR_TC_MAX : (tc < 1 ? 1 : tc);
}

template <int DS>
__global__ void gated_recurrence_kernel(GatedRecurrenceParams p) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x >> 5) - GR_FEED;     // computing warps
  const int dimp = nwarps * DS;
  const int tc = gr_chunk_tokens(dimp);
  const int buf_floats = tc * (2 * dimp + 32);        // one buffer: f [tc][dimp], q [tc][dimp], v [tc][32]
  const int part_floats = tc * nwarps * 32;           // one buffer of shares: [tc][nwarps][32]
  float* bufs = smem;
  float* parts = smem + 2 * buf_floats;
  const int h = blockIdx.y, seq = blockIdx.z, e0 = blockIdx.x * 32;
  const int first = p.cu_tokens[seq], n = p.cu_tokens[seq + 1] - first;
  const int chunks = (n + tc - 1) / tc;
  const bool feeder = warp >= nwarps;
  const int ft = threadIdx.x - nwarps * 32;           // index among the feeding threads

  // What a feeding thread makes of every chunk: gate values u = 0..7 at (token tt[u] of the chunk, row d[u]),
  // and values v at up to two (token, column) places.  The places, the bias and the lower bound do not change
  // from chunk to chunk.
  int g_tt[GR_PER], g_d[GR_PER];
  float g_bias[GR_PER], g_low[GR_PER];
  float a[GR_PER], b[GR_PER], vv[2];
  if (feeder) {
#pragma unroll
    for (int u = 0; u < GR_PER; ++u) {
      const int idx = u * GR_FT + ft;
      g_tt[u] = idx / dimp; g_d[u] = idx - g_tt[u] * dimp;
      const bool real = g_tt[u] < tc && g_d[u] < p.dim;
      g_bias[u] = real ? p.bias[h * p.dim + g_d[u]] : 0.f;
      g_low[u] = real ? p.lower[h * p.dim + g_d[u]] : 1.f;    // rows beyond dim: f = 1, q = 0, the state stays zero
      a[u] = 0.f; b[u] = 0.f;
    }
    vv[0] = vv[1] = 0.f;
  }
  pdl_wait();
  auto request = [&](int cs) {                        // the inputs of chunk cs, into registers
    const int c0 = cs * tc, cn = min(tc, n - c0);
#pragma unroll
    for (int u = 0; u < GR_PER; ++u) {
      a[u] = 0.f; b[u] = 0.f;
      if (g_tt[u] < cn && g_d[u] < p.dim) {
        const float* row = p.pre + (size_t)(first + c0 + g_tt[u]) * p.ld + h * p.dim + g_d[u];
        a[u] = row[p.q_col];
        b[u] = row[p.f_col];
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int idx = u * GR_FT + ft, tt = idx >> 5, ee = e0 + (idx & 31);
      vv[u] = (tt < cn && ee < p.vdim) ? p.pre[(size_t)(first + c0 + tt) * p.ld + p.v_col + h * p.vdim + ee] : 0.f;
    }
  };

  float s[DS];
  float* st = p.state + (((size_t)p.slots[seq] * p.heads + h) * p.dim) * p.vdim;
  const int e = e0 + lane;
  const bool e_ok = e < p.vdim;
  if (!feeder) {
#pragma unroll
    for (int i = 0; i < DS; ++i) {
      const int d = warp * DS + i;
      s[i] = (d < p.dim && e_ok) ? st[(size_t)d * p.vdim + e] : 0.f;
    }
  } else if (chunks > 0) {
    request(0);
  }
  // iteration c: the computing warps walk chunk c; the feeding warps stage chunk c + 1, request chunk c + 2 and
  // finish chunk c - 1
  for (int c = -1; c <= chunks; ++c) {
    if (feeder) {
      const int cs = c + 1;
      if (cs < chunks) {
        float* fs = bufs + (cs & 1) * buf_floats;
        float* qs = fs + tc * dimp;
        float* vs = qs + tc * dimp;
#pragma unroll
        for (int u = 0; u < GR_PER; ++u) {
          if (g_tt[u] < tc) {
            const float x = b[u] + g_bias[u];
            qs[u * GR_FT + ft] = a[u] / (1.f + expf(-a[u]));
            fs[u * GR_FT + ft] = g_low[u] + (1.f - g_low[u]) * (1.f / (1.f + expf(-x)));
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
          if (u * GR_FT + ft < tc * 32) vs[u * GR_FT + ft] = vv[u];
        if (cs + 1 < chunks) request(cs + 1);
      }
      const int cr = c - 1;
      if (cr >= 0) {
        const float* part = parts + (cr & 1) * part_floats;
        const int c0 = cr * tc, cn = min(tc, n - c0);
        for (int idx = ft; idx < cn * 32; idx += GR_FT) {
          const int tt = idx >> 5, l = idx & 31, ee = e0 + l;
          if (ee >= p.vdim) continue;
          float o = 0.f;
          for (int w = 0; w < nwarps; ++w) o += part[(tt * nwarps + w) * 32 + l];
          p.out[(size_t)(first + c0 + tt) * (p.heads * p.vdim) + h * p.vdim + ee] = o;
        }
      }
    } else if (c >= 0 && c < chunks) {
      const float* fs = bufs + (c & 1) * buf_floats;
      const float* qs = fs + tc * dimp;
      const float* vs = qs + tc * dimp;
      float* part = parts + (c & 1) * part_floats;
      const int cn = min(tc, n - c * tc);
      for (int tt = 0; tt < cn; ++tt) {
        const float v = vs[tt * 32 + lane];
        const float* fr = fs + tt * dimp + warp * DS;
        const float* qr = qs + tt * dimp + warp * DS;
        float acc = 0.f;                              // rows in order: the sum does not depend on the schedule
        // f s + (1 - f) v as v + f (s - v): one subtraction and one fused multiply-add a row
#pragma unroll
        for (int i4 = 0; i4 < DS; i4 += 4) {
          const float4 f4 = *reinterpret_cast<const float4*>(fr + i4);
          const float4 q4 = *reinterpret_cast<const float4*>(qr + i4);
          s[i4 + 0] = fmaf(f4.x, s[i4 + 0] - v, v); acc = fmaf(s[i4 + 0], q4.x, acc);
          s[i4 + 1] = fmaf(f4.y, s[i4 + 1] - v, v); acc = fmaf(s[i4 + 1], q4.y, acc);
          s[i4 + 2] = fmaf(f4.z, s[i4 + 2] - v, v); acc = fmaf(s[i4 + 2], q4.z, acc);
          s[i4 + 3] = fmaf(f4.w, s[i4 + 3] - v, v); acc = fmaf(s[i4 + 3], q4.w, acc);
        }
        part[(tt * nwarps + warp) * 32 + lane] = acc;
      }
    }
    __syncthreads();
  }
  if (!feeder) {
#pragma unroll
    for (int i = 0; i < DS; ++i) {
      const int d = warp * DS + i;
      if (d < p.dim && e_ok) st[(size_t)d * p.vdim + e] = s[i];
    }
  }
}

template <int DS>
static cudaError_t launch_gated_recurrence(const GatedRecurrenceParams& p, int num_seqs, cudaStream_t stream) {
  const int nwarps = (p.dim + DS - 1) / DS;
  const int tc = gr_chunk_tokens(nwarps * DS);
  const size_t smem = (size_t)(2 * tc * (2 * nwarps * DS + 32) + 2 * tc * nwarps * 32) * sizeof(float);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    const cudaError_t e = cudaFuncSetAttribute(gated_recurrence_kernel<DS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    allowed = smem;
  }
  return launch(gated_recurrence_kernel<DS>, dim3((p.vdim + 31) / 32, p.heads, num_seqs), dim3((nwarps + GR_FEED) * 32), smem, stream, p);
}

// The same for steps in which no sequence brings more than a few tokens (decoding): no feeding warps and few
// registers, so that several CTAs share an SM while each streams its part of the state in and out, which is all
// the time such a step takes.  Every warp stages the (few) tokens, then walks them, then the shares are added in
// warp order: the sums and their order are those of the kernel above, so both give the same bits.
constexpr int GR_SHORT_TC = 4;

template <int DS, int MAX_THREADS>
__global__ void __launch_bounds__(MAX_THREADS) gated_recurrence_short_kernel(GatedRecurrenceParams p) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int dimp = nwarps * DS;
  float* fs = smem;                                   // [TC][dimp]
  float* qs = fs + GR_SHORT_TC * dimp;                // [TC][dimp]
  float* vs = qs + GR_SHORT_TC * dimp;                // [TC][32]
  float* part = vs + GR_SHORT_TC * 32;                // [TC][nwarps][32]
  const int e = blockIdx.x * 32 + lane, h = blockIdx.y, seq = blockIdx.z;
  const bool e_ok = e < p.vdim;
  const int first = p.cu_tokens[seq], n = p.cu_tokens[seq + 1] - first;
  float* st = p.state + (((size_t)p.slots[seq] * p.heads + h) * p.dim) * p.vdim;
  float s[DS];
  pdl_wait();
#pragma unroll
  for (int i = 0; i < DS; ++i) {
    const int d = warp * DS + i;
    s[i] = (d < p.dim && e_ok) ? st[(size_t)d * p.vdim + e] : 0.f;
  }
  for (int c0 = 0; c0 < n; c0 += GR_SHORT_TC) {
    const int cn = min(GR_SHORT_TC, n - c0);
    for (int idx = threadIdx.x; idx < cn * dimp; idx += blockDim.x) {
      const int tt = idx / dimp, d = idx - tt * dimp;
      float f = 1.f, q = 0.f;
      if (d < p.dim) {
        const float* row = p.pre + (size_t)(first + c0 + tt) * p.ld;
        const int hd = h * p.dim + d;
        const float a = row[p.q_col + hd];
        const float x = row[p.f_col + hd] + p.bias[hd];
        const float low = p.lower[hd];
        q = a / (1.f + expf(-a));
        f = low + (1.f - low) * (1.f / (1.f + expf(-x)));
      }
      fs[idx] = f; qs[idx] = q;
    }
    for (int idx = threadIdx.x; idx < cn * 32; idx += blockDim.x) {
      const int tt = idx >> 5, ee = blockIdx.x * 32 + (idx & 31);
      vs[idx] = ee < p.vdim ? p.pre[(size_t)(first + c0 + tt) * p.ld + p.v_col + h * p.vdim + ee] : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float v = vs[tt * 32 + lane];
      const float* fr = fs + tt * dimp + warp * DS;
      const float* qr = qs + tt * dimp + warp * DS;
      float acc = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < DS; i4 += 4) {
        const float4 f4 = *reinterpret_cast<const float4*>(fr + i4);
        const float4 q4 = *reinterpret_cast<const float4*>(qr + i4);
        s[i4 + 0] = fmaf(f4.x, s[i4 + 0] - v, v); acc = fmaf(s[i4 + 0], q4.x, acc);
        s[i4 + 1] = fmaf(f4.y, s[i4 + 1] - v, v); acc = fmaf(s[i4 + 1], q4.y, acc);
        s[i4 + 2] = fmaf(f4.z, s[i4 + 2] - v, v); acc = fmaf(s[i4 + 2], q4.z, acc);
        s[i4 + 3] = fmaf(f4.w, s[i4 + 3] - v, v); acc = fmaf(s[i4 + 3], q4.w, acc);
      }
      part[(tt * nwarps + warp) * 32 + lane] = acc;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < cn * 32; idx += blockDim.x) {
      const int tt = idx >> 5, l = idx & 31, ee = blockIdx.x * 32 + l;
      if (ee >= p.vdim) continue;
      float o = 0.f;
      for (int w = 0; w < nwarps; ++w) o += part[(tt * nwarps + w) * 32 + l];
      p.out[(size_t)(first + c0 + tt) * (p.heads * p.vdim) + h * p.vdim + ee] = o;
    }
    // the next chunk's staging writes fs, qs and vs, which nobody reads any more; `part` is written again only
    // behind the barrier that follows that staging
  }
#pragma unroll
  for (int i = 0; i < DS; ++i) {
    const int d = warp * DS + i;
    if (d < p.dim && e_ok) st[(size_t)d * p.vdim + e] = s[i];
  }
}

template <int DS, int MAX_THREADS = 256>
static cudaError_t launch_gated_recurrence_short(const GatedRecurrenceParams& p, int num_seqs, cudaStream_t stream) {
  const int nwarps = (p.dim + DS - 1) / DS;
  const size_t smem = (size_t)GR_SHORT_TC * (2 * nwarps * DS + 32 + nwarps * 32) * sizeof(float);      // up to 50 KB (32 warps)
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    const cudaError_t e = cudaFuncSetAttribute(gated_recurrence_short_kernel<DS, MAX_THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    allowed = smem;
  }
  return launch(gated_recurrence_short_kernel<DS, MAX_THREADS>, dim3((p.vdim + 31) / 32, p.heads, num_seqs), dim3(nwarps * 32), smem, stream, p);
}

}  // namespace lb

LB_EXPORT int lb_gated_recurrence(const float* pre, long long ld, int q_col, int f_col, int v_col, const float* bias,
                                  const float* lower, float* state, float* out, const int* cu_tokens, const int* slots,
                                  int num_seqs, int heads, int dim, int vdim, int max_tokens_a_seq, cudaStream_t stream) {
  LB_CHECK_ARG(pre && bias && lower && state && out && cu_tokens && slots, "gated_recurrence: null argument");
  LB_CHECK_ARG(num_seqs >= 0 && heads > 0 && heads <= 65535 && dim > 0 && dim <= 1024 && vdim > 0 && num_seqs <= 65535,
               "gated_recurrence: bad sizes seqs=%d heads=%d dim=%d vdim=%d (dim at most 1024)", num_seqs, heads, dim, vdim);
  if (num_seqs == 0) return 0;
  lb::GatedRecurrenceParams p;
  p.pre = pre; p.ld = ld; p.q_col = q_col; p.f_col = f_col; p.v_col = v_col; p.bias = bias; p.lower = lower;
  p.state = state; p.out = out; p.cu_tokens = cu_tokens; p.slots = slots; p.heads = heads; p.dim = dim; p.vdim = vdim;
  cudaError_t e;
  // rows of the state a warp keeps: as few as give at most 8 warps.  Heads of more than 256 rows: 32 rows a warp and
  // up to 32 warps, in the kernel without feeding warps whatever the step (the other would need more registers than a
  // CTA of that size can have).
  if (dim > 256) e = lb::launch_gated_recurrence_short<32, 1024>(p, num_seqs, stream);
  else if (max_tokens_a_seq > 0 && max_tokens_a_seq <= lb::GR_SHORT_TC) {
    if (dim <= 32) e = lb::launch_gated_recurrence_short<4>(p, num_seqs, stream);
    else if (dim <= 64) e = lb::launch_gated_recurrence_short<8>(p, num_seqs, stream);
    else if (dim <= 128) e = lb::launch_gated_recurrence_short<16>(p, num_seqs, stream);
    else e = lb::launch_gated_recurrence_short<32>(p, num_seqs, stream);
  } else if (dim <= 32) e = lb::launch_gated_recurrence<4>(p, num_seqs, stream);
  else if (dim <= 64) e = lb::launch_gated_recurrence<8>(p, num_seqs, stream);
  else if (dim <= 128) e = lb::launch_gated_recurrence<16>(p, num_seqs, stream);
  else e = lb::launch_gated_recurrence<32>(p, num_seqs, stream);
  if (e != cudaSuccess) { lb::set_error("gated_recurrence: %s", cudaGetErrorString(e)); return 2; }
  LB_CHECK_LAUNCH("gated_recurrence");
  return 0;
}
