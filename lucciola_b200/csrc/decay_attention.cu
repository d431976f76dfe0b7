// Linear attention with a fixed decay per head ("lightning attention"): per sequence and head, with a state
// S [dim, vdim] in 32-bit,
//
//   q_t = silu(a_t)   k_t = silu(b_t)   v_t = silu(c_t)        a, b, c: this token's columns of the input projection
//   S_t = decay_h * S_(t-1) + k_t v_t^T
//   o_t = S_t^T q_t
//
// for the tokens of a step, which are portions of several sequences; a sequence's state is read from its slot
// before its first token of the step and written back after its last.  Everything here is 32-bit, and the
// state is carried token by token: no chunk is multiplied out, so nothing is divided by a power of the decay.
//
// One CTA takes (32 value columns, one head, one sequence).  Warp w keeps rows w*DS .. w*DS+DS-1 of the state
// in registers, one value column a lane.  The tokens are walked in chunks: all threads turn a chunk's inputs into
// q, k and v in shared memory, then every warp walks the chunk's tokens in order and leaves its share of o_t,
// and the shares are added in warp order.  The order of every sum is fixed by (dim, DS) alone, so a token's
// result does not depend on how the sequence was cut into steps or on what else is in the batch.
//
// Also here: what follows the recurrence in a mixer of this kind (the heads' outputs normed together, gated
// elementwise) and the gate of one number a head that a softmax attention beside it may have.
#include "common.cuh"

namespace lb {

struct DecayRecurrenceParams {
  const float* pre; long long ld;       // [T, ld]: q pre-activations at q_col, k at k_col, v at v_col
  int q_col, k_col, v_col;
  const float* decay;                   // [heads]
  float* state;                         // [slots + 1, heads, dim, vdim]
  float* out;                           // [T, heads * vdim]
  const int* cu_tokens; const int* slots;
  int heads, dim, vdim;
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

template <int DS, int TC, int MAX_THREADS>
__global__ void __launch_bounds__(MAX_THREADS) decay_recurrence_kernel(DecayRecurrenceParams p) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int dimp = nwarps * DS;
  float* ks = smem;                                   // [TC][dimp]
  float* qs = ks + TC * dimp;                         // [TC][dimp]
  float* vs = qs + TC * dimp;                         // [TC][32]
  float* part = vs + TC * 32;                         // [TC][nwarps][32]
  const int e = blockIdx.x * 32 + lane, h = blockIdx.y, seq = blockIdx.z;
  const bool e_ok = e < p.vdim;
  const float decay = p.decay[h];
  const int first = p.cu_tokens[seq], n = p.cu_tokens[seq + 1] - first;
  float* st = p.state + (((size_t)p.slots[seq] * p.heads + h) * p.dim) * p.vdim;
  float s[DS];
  pdl_wait();
#pragma unroll
  for (int i = 0; i < DS; ++i) {
    const int d = warp * DS + i;
    s[i] = (d < p.dim && e_ok) ? st[(size_t)d * p.vdim + e] : 0.f;
  }
  for (int c0 = 0; c0 < n; c0 += TC) {
    const int cn = min(TC, n - c0);
    for (int idx = threadIdx.x; idx < cn * dimp; idx += blockDim.x) {
      const int tt = idx / dimp, d = idx - tt * dimp;
      float k = 0.f, q = 0.f;                         // rows beyond dim: nothing enters, nothing is read
      if (d < p.dim) {
        const float* row = p.pre + (size_t)(first + c0 + tt) * p.ld + h * p.dim + d;
        q = silu_f(row[p.q_col]);
        k = silu_f(row[p.k_col]);
      }
      ks[idx] = k; qs[idx] = q;
    }
    for (int idx = threadIdx.x; idx < cn * 32; idx += blockDim.x) {
      const int tt = idx >> 5, ee = blockIdx.x * 32 + (idx & 31);
      vs[idx] = ee < p.vdim ? silu_f(p.pre[(size_t)(first + c0 + tt) * p.ld + p.v_col + h * p.vdim + ee]) : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float v = vs[tt * 32 + lane];
      const float* kr = ks + tt * dimp + warp * DS;
      const float* qr = qs + tt * dimp + warp * DS;
      float acc = 0.f;                                // rows in order
#pragma unroll
      for (int i4 = 0; i4 < DS; i4 += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kr + i4);
        const float4 q4 = *reinterpret_cast<const float4*>(qr + i4);
        s[i4 + 0] = fmaf(decay, s[i4 + 0], k4.x * v); acc = fmaf(s[i4 + 0], q4.x, acc);
        s[i4 + 1] = fmaf(decay, s[i4 + 1], k4.y * v); acc = fmaf(s[i4 + 1], q4.y, acc);
        s[i4 + 2] = fmaf(decay, s[i4 + 2], k4.z * v); acc = fmaf(s[i4 + 2], q4.z, acc);
        s[i4 + 3] = fmaf(decay, s[i4 + 3], k4.w * v); acc = fmaf(s[i4 + 3], q4.w, acc);
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
    // the next chunk's staging writes ks, qs and vs, which nobody reads any more; `part` is written again only
    // behind the barrier that follows that staging
  }
#pragma unroll
  for (int i = 0; i < DS; ++i) {
    const int d = warp * DS + i;
    if (d < p.dim && e_ok) st[(size_t)d * p.vdim + e] = s[i];
  }
}

template <int DS, int TC, int MAX_THREADS = 256>
static cudaError_t launch_decay_recurrence(const DecayRecurrenceParams& p, int num_seqs, cudaStream_t stream) {
  const int nwarps = (p.dim + DS - 1) / DS;
  const size_t smem = (size_t)TC * (2 * nwarps * DS + 32 + nwarps * 32) * sizeof(float);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    const cudaError_t e = cudaFuncSetAttribute(decay_recurrence_kernel<DS, TC, MAX_THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    allowed = smem;
  }
  return launch(decay_recurrence_kernel<DS, TC, MAX_THREADS>, dim3((p.vdim + 31) / 32, p.heads, num_seqs), dim3(nwarps * 32), smem, stream, p);
}

// out[t, :] = x[t, :] * rsqrt(mean(x[t]^2) + eps) * weight * sigmoid(gate[t, :]) * scale: the heads' outputs normed
// together and gated elementwise.  out may be a column range of a wider matrix (row stride out_ld).
template <typename TO>
__global__ void rmsnorm_gated_kernel(TO* __restrict__ out, long long out_ld, const float* __restrict__ x,
                                     const float* __restrict__ weight, const float* __restrict__ gate, long long gate_ld,
                                     float scale, float eps, int n) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const float* r = x + (size_t)blockIdx.x * n;
  const float* g = gate + (size_t)blockIdx.x * gate_ld;
  float ss = 0.f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) ss += r[j] * r[j];
  const float inv = rsqrtf(block_sum(ss, scratch) / (float)n + eps);
  TO* o = out + (size_t)blockIdx.x * out_ld;
  for (int j = threadIdx.x; j < n; j += blockDim.x)
    o[j] = from_f32<TO>(r[j] * inv * weight[j] * (1.f / (1.f + expf(-g[j]))) * scale);
}

// out[t, h, :] = x[t, h, :] * sigmoid(gate[t, h]) * scale: one number a head
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, long long out_ld, const T* __restrict__ x, const float* __restrict__ gate,
                                 long long gate_ld, float scale, int heads, int vdim) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, n = heads * vdim;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float g = gate[(size_t)t * gate_ld + j / vdim];
    out[(size_t)t * out_ld + j] = from_f32<T>(to_f32(x[(size_t)t * n + j]) * (1.f / (1.f + expf(-g))) * scale);
  }
}

}  // namespace lb

// max_tokens_a_seq: the most tokens any sequence brings, if the host knows it (0: unknown); it only chooses the
// chunk's size, which never shows in a result.
LB_EXPORT int lb_decay_recurrence(const float* pre, long long ld, int q_col, int k_col, int v_col, const float* decay,
                                  float* state, float* out, const int* cu_tokens, const int* slots, int num_seqs,
                                  int heads, int dim, int vdim, int max_tokens_a_seq, cudaStream_t stream) {
  LB_CHECK_ARG(pre && decay && state && out && cu_tokens && slots, "decay_recurrence: null argument");
  LB_CHECK_ARG(num_seqs >= 0 && heads > 0 && heads <= 65535 && dim > 0 && dim <= 1024 && vdim > 0 && num_seqs <= 65535,
               "decay_recurrence: bad sizes seqs=%d heads=%d dim=%d vdim=%d (dim at most 1024)", num_seqs, heads, dim, vdim);
  if (num_seqs == 0) return 0;
  lb::DecayRecurrenceParams p;
  p.pre = pre; p.ld = ld; p.q_col = q_col; p.k_col = k_col; p.v_col = v_col; p.decay = decay;
  p.state = state; p.out = out; p.cu_tokens = cu_tokens; p.slots = slots; p.heads = heads; p.dim = dim; p.vdim = vdim;
  const bool few = max_tokens_a_seq > 0 && max_tokens_a_seq <= 4;
  cudaError_t e;
  // rows of the state a warp keeps: as few as give at most 8 warps; heads of more than 256 rows: 32 rows a warp
  if (dim > 256) e = lb::launch_decay_recurrence<32, 4, 1024>(p, num_seqs, stream);
  else if (few) {
    if (dim <= 32) e = lb::launch_decay_recurrence<4, 4>(p, num_seqs, stream);
    else if (dim <= 64) e = lb::launch_decay_recurrence<8, 4>(p, num_seqs, stream);
    else if (dim <= 128) e = lb::launch_decay_recurrence<16, 4>(p, num_seqs, stream);
    else e = lb::launch_decay_recurrence<32, 4>(p, num_seqs, stream);
  } else if (dim <= 32) e = lb::launch_decay_recurrence<4, 16>(p, num_seqs, stream);
  else if (dim <= 64) e = lb::launch_decay_recurrence<8, 16>(p, num_seqs, stream);
  else if (dim <= 128) e = lb::launch_decay_recurrence<16, 16>(p, num_seqs, stream);
  else e = lb::launch_decay_recurrence<32, 16>(p, num_seqs, stream);
  if (e != cudaSuccess) { lb::set_error("decay_recurrence: %s", cudaGetErrorString(e)); return 2; }
  LB_CHECK_LAUNCH("decay_recurrence");
  return 0;
}

LB_EXPORT int lb_rmsnorm_gated(void* out, int out_dtype, long long out_ld, const float* x, const float* weight,
                               const float* gate, long long gate_ld, float scale, float eps, int num_rows, int n,
                               cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && out && x && weight && gate, "rmsnorm_gated: bad arguments");
  LB_CHECK_ARG(num_rows >= 0 && n > 0 && out_ld >= n && gate_ld >= n, "rmsnorm_gated: bad sizes rows=%d n=%d", num_rows, n);
  if (num_rows == 0) return 0;
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  LB_DISPATCH_DTYPE(out_dtype, TO, {
    lb::launch(lb::rmsnorm_gated_kernel<TO>, dim3(num_rows), dim3(threads), 0, stream, (TO*)out, out_ld, x, weight, gate, gate_ld,
               scale, eps, n);
  })
  LB_CHECK_LAUNCH("rmsnorm_gated");
  return 0;
}

LB_EXPORT int lb_head_gate(void* out, int dtype, long long out_ld, const void* x, const float* gate, long long gate_ld,
                           float scale, int num_rows, int heads, int vdim, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(dtype) && out && x && gate, "head_gate: bad arguments");
  LB_CHECK_ARG(num_rows >= 0 && heads > 0 && vdim > 0 && out_ld >= (long long)heads * vdim && gate_ld >= heads,
               "head_gate: bad sizes rows=%d heads=%d vdim=%d", num_rows, heads, vdim);
  if (num_rows == 0) return 0;
  const int n = heads * vdim;
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  LB_DISPATCH_DTYPE(dtype, T, {
    lb::launch(lb::head_gate_kernel<T>, dim3(num_rows), dim3(threads), 0, stream, (T*)out, out_ld, (const T*)x, gate, gate_ld, scale,
               heads, vdim);
  })
  LB_CHECK_LAUNCH("head_gate");
  return 0;
}
