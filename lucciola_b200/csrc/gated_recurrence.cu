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
// One CTA takes (32 value columns, one head, one sequence).  Warp w keeps rows w*DS .. w*DS+DS-1 of the
// state in registers, one value column a lane, and walks the tokens in order.  Tokens are staged in chunks
// of TC: the gates of the chunk are computed once into shared memory, every warp leaves its rows' share of
// o_t there, and after the chunk the shares are added in warp order: the order of every sum is fixed by
// (dim, DS) alone, so a token's result does not depend on how the sequence was cut into steps.
#include "common.cuh"

namespace lb {

constexpr int GR_TC = 16;

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
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int dimp = nwarps * DS;
  float* fs = smem;                                   // [TC][dimp]
  float* qs = fs + GR_TC * dimp;                      // [TC][dimp]
  float* vs = qs + GR_TC * dimp;                      // [TC][32]
  float* part = vs + GR_TC * 32;                      // [TC][nwarps][32]
  const int e = blockIdx.x * 32 + lane, h = blockIdx.y, seq = blockIdx.z;
  const bool e_ok = e < p.vdim;
  const int first = p.cu_tokens[seq], n = p.cu_tokens[seq + 1] - first;
  pdl_wait();
  float* st = p.state + (((size_t)p.slots[seq] * p.heads + h) * p.dim) * p.vdim;
  float s[DS];
#pragma unroll
  for (int i = 0; i < DS; ++i) {
    const int d = warp * DS + i;
    s[i] = (d < p.dim && e_ok) ? st[(size_t)d * p.vdim + e] : 0.f;
  }
  for (int c0 = 0; c0 < n; c0 += GR_TC) {
    const int cn = min(GR_TC, n - c0);
    for (int idx = threadIdx.x; idx < cn * dimp; idx += blockDim.x) {
      const int tt = idx / dimp, d = idx - tt * dimp;
      float f = 1.f, q = 0.f;                         // rows beyond dim: the state stays zero
      if (d < p.dim) {
        const float* row = p.pre + (size_t)(first + c0 + tt) * p.ld;
        const int hd = h * p.dim + d;
        const float a = row[p.q_col + hd];
        q = a / (1.f + expf(-a));
        const float g = 1.f / (1.f + expf(-(row[p.f_col + hd] + p.bias[hd])));
        const float low = p.lower[hd];
        f = low + (1.f - low) * g;
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
        s[i4 + 0] = f4.x * s[i4 + 0] + (1.f - f4.x) * v; acc = fmaf(s[i4 + 0], q4.x, acc);
        s[i4 + 1] = f4.y * s[i4 + 1] + (1.f - f4.y) * v; acc = fmaf(s[i4 + 1], q4.y, acc);
        s[i4 + 2] = f4.z * s[i4 + 2] + (1.f - f4.z) * v; acc = fmaf(s[i4 + 2], q4.z, acc);
        s[i4 + 3] = f4.w * s[i4 + 3] + (1.f - f4.w) * v; acc = fmaf(s[i4 + 3], q4.w, acc);
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
    // the next chunk's staging writes fs, qs and vs, which nobody reads any more; `part` is written again
    // only behind the barrier that follows that staging
  }
#pragma unroll
  for (int i = 0; i < DS; ++i) {
    const int d = warp * DS + i;
    if (d < p.dim && e_ok) st[(size_t)d * p.vdim + e] = s[i];
  }
}

template <int DS>
static cudaError_t launch_gated_recurrence(const GatedRecurrenceParams& p, int num_seqs, cudaStream_t stream) {
  const int nwarps = (p.dim + DS - 1) / DS;
  const size_t smem = (size_t)GR_TC * (2 * nwarps * DS + 32 + nwarps * 32) * sizeof(float);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    const cudaError_t e = cudaFuncSetAttribute(gated_recurrence_kernel<DS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    allowed = smem;
  }
  return launch(gated_recurrence_kernel<DS>, dim3((p.vdim + 31) / 32, p.heads, num_seqs), dim3(nwarps * 32), smem, stream, p);
}

}  // namespace lb

LB_EXPORT int lb_gated_recurrence(const float* pre, long long ld, int q_col, int f_col, int v_col, const float* bias,
                                  const float* lower, float* state, float* out, const int* cu_tokens, const int* slots,
                                  int num_seqs, int heads, int dim, int vdim, cudaStream_t stream) {
  LB_CHECK_ARG(pre && bias && lower && state && out && cu_tokens && slots, "gated_recurrence: null argument");
  LB_CHECK_ARG(num_seqs >= 0 && heads > 0 && heads <= 65535 && dim > 0 && dim <= 1024 && vdim > 0 && num_seqs <= 65535,
               "gated_recurrence: bad sizes seqs=%d heads=%d dim=%d vdim=%d (dim at most 1024)", num_seqs, heads, dim, vdim);
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
