// A short causal convolution over time on each channel, added to its input:
//
//   out_t = h_t + sum_{j < taps} w[:, j] * h_(t - taps + 1 + j)        (zeros before the sequence's start)
//
// for the tokens of a step, which are portions of several sequences.  What lies before a portion comes
// from the sequence's state: the last taps - 1 inputs, oldest first, [slots + 1, taps - 1, width], zero
// for a new sequence.  lb_causal_taps reads the state; lb_causal_taps_state, launched after it, replaces
// the state by the last taps - 1 inputs of (state ++ portion).  Products and sums are 32-bit; the weight comes
// transposed, [taps, width] in 32-bit (oldest tap first), so that neighbouring channels read neighbouring words.
#include "common.cuh"

namespace lb {

constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void causal_taps_kernel(T* __restrict__ out, const T* __restrict__ h, const float* __restrict__ w,
                                   const T* __restrict__ state, const int* __restrict__ token_seq,
                                   const int* __restrict__ cu_tokens, const int* __restrict__ slots, int width, int taps) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  const int idx = t - cu_tokens[s];                       // place of the token in its portion
  const T* st = state ? state + (size_t)slots[s] * (taps - 1) * width : nullptr;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps - 1; ++j) {                  // the input taps - 1 - j tokens back
      const int back = taps - 1 - j;
      float v;
      if (idx - back >= 0) v = to_f32(h[(size_t)(t - back) * width + c]);
      else v = to_f32(st[(size_t)(taps - 1 + idx - back) * width + c]);
      acc = fmaf(w[(size_t)j * width + c], v, acc);
    }
    const float cur = to_f32(h[(size_t)t * width + c]);
    acc = fmaf(w[(size_t)(taps - 1) * width + c], cur, acc);
    out[(size_t)t * width + c] = from_f32<T>(cur + acc);
  }
}

// The same for bfloat16 rows whose width is a multiple of 8: eight channels a thread, 16-byte accesses.
__global__ void causal_taps_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ h, const float* __restrict__ w,
                                          const bf16* __restrict__ state, const int* __restrict__ token_seq,
                                          const int* __restrict__ cu_tokens, const int* __restrict__ slots, int width, int taps) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  const int idx = t - cu_tokens[s];
  const bf16* st = state ? state + (size_t)slots[s] * (taps - 1) * width : nullptr;
  for (int c = 8 * (blockIdx.y * blockDim.x + threadIdx.x); c < width; c += 8 * gridDim.y * blockDim.x) {
    float acc[8], cur[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      const bf16* src = idx - back >= 0 ? h + (size_t)(t - back) * width + c : st + (size_t)(taps - 1 + idx - back) * width + c;
      const uint4 raw = *reinterpret_cast<const uint4*>(src);
      const float4 wa = *reinterpret_cast<const float4*>(w + (size_t)j * width + c);
      const float4 wb = *reinterpret_cast<const float4*>(w + (size_t)j * width + c + 4);
      const float wk[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 x = __bfloat1622float2(p2[k]);
        cur[2 * k] = x.x; cur[2 * k + 1] = x.y;                 // after the last tap: the token's own input
        acc[2 * k] = fmaf(wk[2 * k], x.x, acc[2 * k]);
        acc[2 * k + 1] = fmaf(wk[2 * k + 1], x.y, acc[2 * k + 1]);
      }
    }
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) o2[k] = __floats2bfloat162_rn(cur[2 * k] + acc[2 * k], cur[2 * k + 1] + acc[2 * k + 1]);
    *reinterpret_cast<uint4*>(out + (size_t)t * width + c) = o4;
  }
}

template <typename T>
__global__ void causal_taps_state_kernel(T* __restrict__ state, const T* __restrict__ h, const int* __restrict__ cu_tokens,
                                         const int* __restrict__ slots, int width, int taps) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x;
  const int first = cu_tokens[s], n = cu_tokens[s + 1] - first;
  T* st = state + (size_t)slots[s] * (taps - 1) * width;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    // entry i of the new state is element n - (taps - 1) + i of the portion, or, where that lies before the
    // portion, entry i + n of the old state; i ascends, so an old entry is read before it is overwritten
    for (int i = 0; i < taps - 1; ++i) {
      const int m = n - (taps - 1) + i;
      st[(size_t)i * width + c] = m >= 0 ? h[(size_t)(first + m) * width + c] : st[(size_t)(i + n) * width + c];
    }
  }
}

}  // namespace lb

LB_EXPORT int lb_causal_taps(int dtype, void* out, const void* h, const float* w, const void* state, const int* token_seq,
                             const int* cu_tokens, const int* slots, int num_tokens, int width, int taps,
                             cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(dtype), "causal_taps: bad dtype %d", dtype);
  LB_CHECK_ARG(num_tokens >= 0 && width > 0 && taps >= 1 && taps <= lb::MAX_TAPS, "causal_taps: bad sizes T=%d width=%d taps=%d",
               num_tokens, width, taps);
  LB_CHECK_ARG(taps == 1 || (state && slots), "causal_taps: more than one tap needs the sequences' state");
  LB_CHECK_ARG(out && h && w && token_seq && cu_tokens, "causal_taps: null argument");
  if (num_tokens == 0) return 0;
  if (dtype == LB_BF16 && width % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)state % 16 == 0 &&
      (uintptr_t)w % 16 == 0) {
    const int threads = width >= 1024 ? 128 : 32;
    int by = (width / 8 + threads - 1) / threads;
    if (by > 64) by = 64;
    lb::launch(lb::causal_taps_bf16x8_kernel, dim3(num_tokens, by), dim3(threads), 0, stream, (lb::bf16*)out, (const lb::bf16*)h, w,
               (const lb::bf16*)state, token_seq, cu_tokens, slots, width, taps);
    LB_CHECK_LAUNCH("causal_taps");
    return 0;
  }
  const int threads = width >= 256 ? 256 : 64;
  int by = (width + threads - 1) / threads;
  if (by > 64) by = 64;
  LB_DISPATCH_DTYPE(dtype, T, {
    lb::launch(lb::causal_taps_kernel<T>, dim3(num_tokens, by), dim3(threads), 0, stream, (T*)out, (const T*)h, w,
               (const T*)state, token_seq, cu_tokens, slots, width, taps);
  })
  LB_CHECK_LAUNCH("causal_taps");
  return 0;
}

LB_EXPORT int lb_causal_taps_state(int dtype, void* state, const void* h, const int* cu_tokens, const int* slots,
                                   int num_seqs, int width, int taps, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(dtype), "causal_taps_state: bad dtype %d", dtype);
  LB_CHECK_ARG(num_seqs >= 0 && width > 0 && taps >= 2 && taps <= lb::MAX_TAPS, "causal_taps_state: bad sizes");
  LB_CHECK_ARG(state && h && cu_tokens && slots, "causal_taps_state: null argument");
  if (num_seqs == 0) return 0;
  const int threads = width >= 256 ? 256 : 64;
  int by = (width + threads - 1) / threads;
  if (by > 64) by = 64;
  LB_DISPATCH_DTYPE(dtype, T, {
    lb::launch(lb::causal_taps_state_kernel<T>, dim3(num_seqs, by), dim3(threads), 0, stream, (T*)state, (const T*)h,
               cu_tokens, slots, width, taps);
  })
  LB_CHECK_LAUNCH("causal_taps_state");
  return 0;
}
