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
// feed them: while the computing warps work on one chunk of TC tokens, the feeding warps form the gates of the
// next chunk in shared memory (two buffers) and add up, in warp order, the shares of o_t that the computing
// warps left for the chunk before; one barrier a chunk.  The order of every sum is fixed by (dim, DS) alone,
// so a token's result does not depend on how the sequence was cut into steps.
#include "common.cuh"

namespace lb {

constexpr int GR_TC = 16;          // tokens a chunk
constexpr int GR_FEED = 8;         // feeding warps

struct GatedRecurrenceParams {
  const float* pre; long long ld;       // [T, ld]: q pre-activations at q_col, gate at f_col, values at v_col
  int q_col, f_col, v_col;
  const float* bias; const float* lower;   // [heads * dim]
  float* state;                         // [slots + 1, heads, dim, vdim]
  float* out;                           // [T, heads * vdim]
  const int* cu_tokens; const int* slots;
  int heads, dim, vdim;
};

template <int DS>
__global__ void gated_recurrence_kernel(GatedRecurrenceParams p) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x >> 5) - GR_FEED;     // computing warps
  const int dimp = nwarps * DS;
  const int buf_floats = GR_TC * (2 * dimp + 32);     // one buffer: f [TC][dimp], q [TC][dimp], v [TC][32]
  const int part_floats = GR_TC * nwarps * 32;        // one buffer of shares: [TC][nwarps][32]
  float* bufs = smem;
  float* parts = smem + 2 * buf_floats;
  const int h = blockIdx.y, seq = blockIdx.z, e0 = blockIdx.x * 32;
  const int first = p.cu_tokens[seq], n = p.cu_tokens[seq + 1] - first;
  const int chunks = (n + GR_TC - 1) / GR_TC;
  const bool feeder = warp >= nwarps;
  pdl_wait();

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
  }
  const int ft = threadIdx.x - nwarps * 32;           // index among the feeding threads
  // iteration c: the computing warps walk chunk c; the feeding warps stage chunk c + 1 and finish chunk c - 1
  for (int c = -1; c <= chunks; ++c) {
    if (feeder) {
      const int cs = c + 1;
      if (cs < chunks) {
        float* fs = bufs + (cs & 1) * buf_floats;
        float* qs = fs + GR_TC * dimp;
        float* vs = qs + GR_TC * dimp;
        const int c0 = cs * GR_TC, cn = min(GR_TC, n - c0);
        // eight elements a thread at a time: all their loads are issued before any is used
        for (int base = 0; base < cn * dimp; base += GR_FEED * 32 * 8) {
          float a[8], b[8], low[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int idx = base + u * GR_FEED * 32 + ft;
            const int tt = idx / dimp, d = idx - tt * dimp;
            a[u] = 0.f; b[u] = 0.f; low[u] = 1.f;          // rows beyond dim: f = 1, q = 0, the state stays zero
            if (idx < cn * dimp && d < p.dim) {
              const float* row = p.pre + (size_t)(first + c0 + tt) * p.ld;
              const int hd = h * p.dim + d;
              a[u] = row[p.q_col + hd];
              b[u] = row[p.f_col + hd] + p.bias[hd];
              low[u] = p.lower[hd];
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int idx = base + u * GR_FEED * 32 + ft;
            if (idx < cn * dimp) {
              qs[idx] = a[u] / (1.f + expf(-a[u]));
              fs[idx] = low[u] + (1.f - low[u]) * (1.f / (1.f + expf(-b[u])));
            }
          }
        }
        for (int idx = ft; idx < cn * 32; idx += GR_FEED * 32) {
          const int tt = idx >> 5, ee = e0 + (idx & 31);
          vs[idx] = ee < p.vdim ? p.pre[(size_t)(first + c0 + tt) * p.ld + p.v_col + h * p.vdim + ee] : 0.f;
        }
      }
      const int cr = c - 1;
      if (cr >= 0) {
        const float* part = parts + (cr & 1) * part_floats;
        const int c0 = cr * GR_TC, cn = min(GR_TC, n - c0);
        for (int idx = ft; idx < cn * 32; idx += GR_FEED * 32) {
          const int tt = idx >> 5, l = idx & 31, ee = e0 + l;
          if (ee >= p.vdim) continue;
          float o = 0.f;
          for (int w = 0; w < nwarps; ++w) o += part[(tt * nwarps + w) * 32 + l];
          p.out[(size_t)(first + c0 + tt) * (p.heads * p.vdim) + h * p.vdim + ee] = o;
        }
      }
    } else if (c >= 0 && c < chunks) {
      const float* fs = bufs + (c & 1) * buf_floats;
      const float* qs = fs + GR_TC * dimp;
      const float* vs = qs + GR_TC * dimp;
      float* part = parts + (c & 1) * part_floats;
      const int cn = min(GR_TC, n - c * GR_TC);
      for (int tt = 0; tt < cn; ++tt) {
        const float v = vs[tt * 32 + lane];
        const float* fr = fs + tt * dimp + warp * DS;
        const float* qr = qs + tt * dimp + warp * DS;
        float acc = 0.f;                              // rows in order: the sum does not depend on the schedule
#pragma unroll
        for (int i4 = 0; i4 < DS; i4 += 4) {
          const float4 f4 = *reinterpret_cast<const float4*>(fr + i4);
          const float4 q4 = *reinterpret_cast<const float4*>(qr + i4);
          s[i4 + 0] = f4.x * s[i4 + 0] + (1.f - f4.x) * v; acc = fmaf(s[i4 + 0], q4.x, acc);
          s[i4 + 1] = f4.y * s[i4 + 1] + (1.f - f4.y) * v; acc = fmaf(s[i4 + 1], q4.y, acc);
          s[i4 + 2] = f4.z * s[i4 + 2] + (1.f - f4.z) * v; acc = fmaf(s[i4 + 2], q4.z, acc);
          s[i4 + 3] = f4.w * s[i4 + 3] + (1.f - f4.w) * v; acc = fmaf(s[i4 + 3], q4.w, acc);
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
  const size_t smem = (size_t)(2 * GR_TC * (2 * nwarps * DS + 32) + 2 * GR_TC * nwarps * 32) * sizeof(float);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    const cudaError_t e = cudaFuncSetAttribute(gated_recurrence_kernel<DS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    allowed = smem;
  }
  return launch(gated_recurrence_kernel<DS>, dim3((p.vdim + 31) / 32, p.heads, num_seqs), dim3((nwarps + GR_FEED) * 32), smem, stream, p);
}

}  // namespace lb

LB_EXPORT int lb_gated_recurrence(const float* pre, long long ld, int q_col, int f_col, int v_col, const float* bias,
                                  const float* lower, float* state, float* out, const int* cu_tokens, const int* slots,
                                  int num_seqs, int heads, int dim, int vdim, cudaStream_t stream) {
  LB_CHECK_ARG(pre && bias && lower && state && out && cu_tokens && slots, "gated_recurrence: null argument");
  LB_CHECK_ARG(num_seqs >= 0 && heads > 0 && heads <= 65535 && dim > 0 && dim <= 768 && vdim > 0 && num_seqs <= 65535,
               "gated_recurrence: bad sizes seqs=%d heads=%d dim=%d vdim=%d (dim at most 768)", num_seqs, heads, dim, vdim);
  if (num_seqs == 0) return 0;
  lb::GatedRecurrenceParams p;
  p.pre = pre; p.ld = ld; p.q_col = q_col; p.f_col = f_col; p.v_col = v_col; p.bias = bias; p.lower = lower;
  p.state = state; p.out = out; p.cu_tokens = cu_tokens; p.slots = slots; p.heads = heads; p.dim = dim; p.vdim = vdim;
  cudaError_t e;
  // rows of the state a warp keeps: as few as give at most 8 warps, 32 from there on
  if (dim <= 32) e = lb::launch_gated_recurrence<4>(p, num_seqs, stream);
  else if (dim <= 64) e = lb::launch_gated_recurrence<8>(p, num_seqs, stream);
  else if (dim <= 128) e = lb::launch_gated_recurrence<16>(p, num_seqs, stream);
  else e = lb::launch_gated_recurrence<32>(p, num_seqs, stream);
  if (e != cudaSuccess) { lb::set_error("gated_recurrence: %s", cudaGetErrorString(e)); return 2; }
  LB_CHECK_LAUNCH("gated_recurrence");
  return 0;
}
