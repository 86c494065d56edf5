// Causal depthwise convolution over time with a few taps, added to its input:
//
//   out[t, c] = h[t, c] + sum_j w[c, j] * h[t - (taps - 1) + j, c]        j = 0 .. taps - 1
//
// (tap taps - 1 multiplies the present input).  Inputs before a request's first
// token are zeros.  The taps - 1 inputs before a step's first token come from the
// request's state, state[slot, i, c] = input at position start - (taps - 1) + i,
// which a new request finds zeroed.  After the step the state holds the last
// taps - 1 inputs again.
//
// Two kernels, because rows of one span read the state that the span's end
// replaces: short_conv_kernel computes every row; short_conv_state_kernel, launched
// after it, moves the state on.  A request that brings a single token has nobody
// else reading its state, so its row moves the state on itself (inline_single), and
// a step of single tokens only needs no second launch.
//
// Products and sums in float32; one thread owns a channel of a row.
#include "common.cuh"

namespace ifx {

constexpr int kMaxTaps = 16;

template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ h, const float* __restrict__ w, float* __restrict__ state,
                                  long long state_slot_stride, const int* __restrict__ token_req,
                                  const int* __restrict__ req_slot, const int* __restrict__ cu_seqlens,
                                  T* __restrict__ out, int channels, int taps, int inline_single) {
  const int t = blockIdx.x;
  const int r = token_req[t];
  const int first = cu_seqlens[r], n = cu_seqlens[r + 1] - first;
  const int i = t - first;                               // index inside the span
  float* st = state ? state + (long long)req_slot[r] * state_slot_stride : nullptr;
  const bool move_on = inline_single && n == 1 && st != nullptr;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    const float* wc = w + (size_t)c * taps;
    const float now = to_f32(h[(size_t)t * channels + c]);
    float acc = fmaf(wc[taps - 1], now, now);
    float older[kMaxTaps - 1];
#pragma unroll
    for (int k = 1; k < kMaxTaps; ++k) {                 // the input k steps back
      if (k < taps) {
        float v;
        if (k <= i) v = to_f32(h[(size_t)(t - k) * channels + c]);
        else v = st[(size_t)((taps - 1) - (k - i)) * channels + c];
        older[k - 1] = v;
        acc = fmaf(wc[taps - 1 - k], v, acc);
      }
    }
    out[(size_t)t * channels + c] = from_f32<T>(acc);
    if (move_on) {                                       // i == 0: older[k - 1] = state[taps - 1 - k]
#pragma unroll
      for (int k = 1; k < kMaxTaps; ++k)
        if (k < taps) st[(size_t)(taps - 1 - k) * channels + c] = (k == 1) ? now : older[k - 2];
    }
  }
}

// New state of request r: the last taps - 1 entries of (old state ++ the span's inputs).
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ h, float* __restrict__ state,
                                        long long state_slot_stride, const int* __restrict__ req_slot,
                                        const int* __restrict__ cu_seqlens, int channels, int taps,
                                        int skip_single) {
  const int r = blockIdx.x;
  const int first = cu_seqlens[r], n = cu_seqlens[r + 1] - first;
  if (skip_single && n == 1) return;
  float* st = state + (long long)req_slot[r] * state_slot_stride;
  const int keep = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float next[kMaxTaps - 1];
#pragma unroll
    for (int s = 0; s < kMaxTaps - 1; ++s) {
      if (s < keep) {
        const int m = n + s;                             // index into old state ++ span
        next[s] = m < keep ? st[(size_t)m * channels + c] : to_f32(h[(size_t)(first + m - keep) * channels + c]);
      }
    }
#pragma unroll
    for (int s = 0; s < kMaxTaps - 1; ++s)
      if (s < keep) st[(size_t)s * channels + c] = next[s];
  }
}

}  // namespace ifx

using namespace ifx;

extern "C" {

// state: float32 [slots, ..., taps - 1, channels], already offset to this convolution's part of a slot;
// state_slot_stride: floats from one slot to the next.  any_long: some request brings more than one token.
int ifx_short_conv(const void* h, const float* w, float* state, long long state_slot_stride, const int* token_req,
                   const int* req_slot, const int* cu_seqlens, void* out, int T, int R, int channels, int taps,
                   int any_long, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (channels <= 0 || taps <= 0 || R <= 0) return IFX_E_BADARG;
  if (taps > kMaxTaps) return IFX_E_TOOBIG;
  if (taps > 1 && state == nullptr) return IFX_E_BADARG;
  const int threads = channels >= 256 ? 256 : ((channels + 31) / 32) * 32;
  const unsigned gy = (unsigned)((channels + threads - 1) / threads);
  if (gy > 65535u) return IFX_E_TOOBIG;
  dim3 grid((unsigned)T, gy), sgrid((unsigned)R, gy);
#define IFX_LAUNCH(TT)                                                                                              \
  do {                                                                                                              \
    short_conv_kernel<TT><<<grid, threads, 0, stream>>>((const TT*)h, w, state, state_slot_stride, token_req,       \
                                                         req_slot, cu_seqlens, (TT*)out, channels, taps, 1);        \
    if (taps > 1 && any_long)                                                                                       \
      short_conv_state_kernel<TT><<<sgrid, threads, 0, stream>>>((const TT*)h, state, state_slot_stride, req_slot,  \
                                                                 cu_seqlens, channels, taps, 1);                    \
  } while (0)
  if (dtype == IFX_DT_F32) IFX_LAUNCH(float);
  else if (dtype == IFX_DT_BF16) IFX_LAUNCH(__nv_bfloat16);
  else return IFX_E_DTYPE;
#undef IFX_LAUNCH
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
