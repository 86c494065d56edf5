// A recurrence with a matrix of state per head (key channels x value channels) and a decay that is made from
// the input, with the small kernels around it.
//
//   token_shift_mix   mixes[m][t] = x[t] + (x[t - 1] - x[t]) * mu[m]      x float32 (the residual stream);
//                     the token before a step's first one is the request's state, zeros at a sequence's start
//   wkv_scan          per request and head, token after token, all in float32:
//                       w_t   = exp(-exp(raw_t + w0))                      decay per key channel
//                       out_t = S^T r_t + (sum_i r_i u_i k_i) v_t          u: a bonus for the present token only
//                       S     = diag(w_t) S + k_t v_t^T
//                     then, per token and head, out / sqrt(mean(out^2) + eps) * norm_w * silu(g) in the run's dtype
//                     S is read from and left in the request's state; so is the step's last input row.
//   cast_rows         float32 -> the run's dtype
//   tanh_rows         z <- tanh(z), in place (the activation inside the decay's two small products)
//
// The scan is sequential in the tokens of a request, so what a position gets does not depend on how the
// tokens were cut into steps: every sum has one order, fixed by the head size alone.
//
// Layout of a thread block of the scan: thread (j, s) owns value channel j and the key channels
// i = s, s + KS, s + 2 KS, ... of S in registers (KS a power of two up to 32; the KS threads of a channel are
// neighbours in a warp and add their shares by shuffles).  r, k, w and v of up to 16 tokens are staged in
// shared memory at a time, so the block synchronises three times per 16 tokens, not per token.
#include "common.cuh"

namespace ifx {

template <typename TO>
__global__ void token_shift_mix_kernel(const float* __restrict__ x, const float* __restrict__ mu,
                                       const float* __restrict__ prev_state, long long slot_stride,
                                       const int* __restrict__ token_req, const int* __restrict__ req_slot,
                                       const int* __restrict__ cu_seqlens, TO* __restrict__ out, int T, int C,
                                       int n_mix) {
  const int t = blockIdx.x;
  const int r = token_req[t];
  const bool first = cu_seqlens[r] == t;
  const float* before = first ? prev_state + (long long)req_slot[r] * slot_stride : x + (size_t)(t - 1) * C;
  const float* now = x + (size_t)t * C;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    const float h = now[i];
    const float dlt = before[i] - h;
    for (int m = 0; m < n_mix; ++m)
      out[((size_t)m * T + t) * C + i] = from_f32<TO>(fmaf(dlt, mu[(size_t)m * C + i], h));
  }
}

template <typename TO>
__global__ void cast_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = from_f32<TO>(x[i]);
}

template <typename T>
__global__ void tanh_rows_kernel(T* __restrict__ z, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    z[i] = from_f32<T>(tanhf(to_f32(z[i])));
}

constexpr int kScanTokens = 16;      // tokens staged at a time

template <int RMAX, typename TO>
__global__ void __launch_bounds__(1024) wkv_scan_kernel(
    const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
    const float* __restrict__ w_raw, const float* __restrict__ g, const float* __restrict__ w0,
    const float* __restrict__ u, const float* __restrict__ norm_w, float eps, float* __restrict__ s_state,
    float* __restrict__ prev_state, long long slot_stride, const float* __restrict__ x, int C,
    const int* __restrict__ cu_seqlens, const int* __restrict__ req_slot, float* __restrict__ o_scratch,
    TO* __restrict__ y, int H, int D, int KS) {
  extern __shared__ float smem[];
  float* r_s = smem;                                 // [kScanTokens][D]
  float* k_s = r_s + kScanTokens * D;
  float* w_s = k_s + kScanTokens * D;
  float* v_s = w_s + kScanTokens * D;
  float* b_s = v_s + kScanTokens * D;                // [kScanTokens] bonus sums
  const int req = blockIdx.x, head = blockIdx.y;
  const int lo = cu_seqlens[req], hi = cu_seqlens[req + 1];
  const int slot = req_slot[req];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int j = tid / KS, s = tid % KS;
  const bool active = j < D;
  const int HD = H * D;
  float* S_g = s_state + (long long)slot * slot_stride + (size_t)head * D * D;
  float S[RMAX];
#pragma unroll
  for (int m = 0; m < RMAX; ++m) {
    const int i = s + KS * m;
    S[m] = (active && i < D) ? S_g[(size_t)i * D + j] : 0.0f;
  }
  for (int t0 = lo; t0 < hi; t0 += kScanTokens) {
    const int nt = min(kScanTokens, hi - t0);
    for (int idx = tid; idx < nt * D; idx += blockDim.x) {
      const int tt = idx / D, i = idx % D;
      const size_t src = (size_t)(t0 + tt) * HD + (size_t)head * D + i;
      r_s[idx] = r[src];
      k_s[idx] = k[src];
      v_s[idx] = v[src];
      w_s[idx] = expf(-expf(w_raw[src] + w0[head * D + i]));
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += nwarps) {       // the bonus of the present token: one number per token
      float b = 0.0f;
      for (int i = lane; i < D; i += 32) b = fmaf(r_s[tt * D + i] * u[head * D + i], k_s[tt * D + i], b);
      b = warp_sum(b);
      if (lane == 0) b_s[tt] = b;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float* rr = r_s + tt * D;
      const float* kk = k_s + tt * D;
      const float* ww = w_s + tt * D;
      const float vj = active ? v_s[tt * D + j] : 0.0f;
      float acc = 0.0f;
#pragma unroll
      for (int m = 0; m < RMAX; ++m) {
        const int i = s + KS * m;
        if (i < D) {
          acc = fmaf(rr[i], S[m], acc);
          S[m] = fmaf(ww[i], S[m], kk[i] * vj);
        }
      }
      for (int o = 1; o < KS; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (active && s == 0) o_scratch[(size_t)(t0 + tt) * HD + (size_t)head * D + j] = fmaf(b_s[tt], vj, acc);
    }
    __syncthreads();
  }
#pragma unroll
  for (int m = 0; m < RMAX; ++m) {
    const int i = s + KS * m;
    if (active && i < D) S_g[(size_t)i * D + j] = S[m];
  }
  if (head == 0 && hi > lo) {                          // the step's last input is the next step's "token before"
    float* p = prev_state + (long long)slot * slot_stride;
    const float* last = x + (size_t)(hi - 1) * C;
    for (int i = tid; i < C; i += blockDim.x) p[i] = last[i];
  }
  // the block's own writes to o_scratch are visible to it after the barrier at the end of the loop
  for (int t = lo + warp; t < hi; t += nwarps) {
    const size_t base = (size_t)t * HD + (size_t)head * D;
    float ss = 0.0f;
    for (int i = lane; i < D; i += 32) {
      const float o = o_scratch[base + i];
      ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)D + eps);
    for (int i = lane; i < D; i += 32) {
      const float gate = g[base + i];
      const float sg = gate / (1.0f + expf(-gate));
      y[base + i] = from_f32<TO>(o_scratch[base + i] * inv * norm_w[head * D + i] * sg);
    }
  }
}

}  // namespace ifx

using namespace ifx;

extern "C" {

int ifx_token_shift_mix(const float* x, const float* mu, const float* prev_state, long long slot_stride,
                        const int* token_req, const int* req_slot, const int* cu_seqlens, void* out, int T, int C,
                        int n_mix, int out_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C <= 0 || n_mix <= 0 || prev_state == nullptr) return IFX_E_BADARG;
  const int threads = C >= 1024 ? 256 : (C >= 256 ? 128 : 64);
  if (out_dtype == IFX_DT_F32)
    token_shift_mix_kernel<float><<<T, threads, 0, stream>>>(x, mu, prev_state, slot_stride, token_req, req_slot,
                                                              cu_seqlens, (float*)out, T, C, n_mix);
  else if (out_dtype == IFX_DT_BF16)
    token_shift_mix_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(x, mu, prev_state, slot_stride, token_req, req_slot,
                                                                      cu_seqlens, (__nv_bfloat16*)out, T, C, n_mix);
  else
    return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_cast_rows(const float* x, void* out, long long n, int out_dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (out_dtype == IFX_DT_F32) cast_rows_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>(x, (float*)out, n);
  else if (out_dtype == IFX_DT_BF16)
    cast_rows_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(x, (__nv_bfloat16*)out, n);
  else return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_tanh_rows(void* z, long long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == IFX_DT_F32) tanh_rows_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((float*)z, n);
  else if (dtype == IFX_DT_BF16) tanh_rows_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((__nv_bfloat16*)z, n);
  else return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

// r, k, v, w_raw, g: float32 [T, H * D].  s_state / prev_state: slot 0's matrix block [H, D, D] and input row [C]
// inside the state tensor, slots slot_stride floats apart.  o_scratch: float32 [T, H * D].  y: [T, H * D].
int ifx_wkv_scan(const float* r, const float* k, const float* v, const float* w_raw, const float* g, const float* w0,
                 const float* u, const float* norm_w, float eps, float* s_state, float* prev_state,
                 long long slot_stride, const float* x, int C, const int* cu_seqlens, const int* req_slot,
                 float* o_scratch, void* y, int num_requests, int H, int D, int out_dtype, cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  if (H <= 0 || D <= 0 || D > 256 || H > 65535) return IFX_E_BADARG;
  int rmax = 16, ks = 1;
  while (ks < 32 && (D + ks - 1) / ks > rmax) ks *= 2;
  if ((D + ks - 1) / ks > rmax || D * ks > 1024) {       // large heads: more of S per thread
    rmax = 64;
    ks = 1;
    while (ks < 32 && (D + ks - 1) / ks > rmax) ks *= 2;
    if ((D + ks - 1) / ks > rmax || D * ks > 1024) return IFX_E_TOOBIG;
  }
  const int threads = (D * ks + 31) / 32 * 32;
  const size_t smem = ((size_t)4 * kScanTokens * D + kScanTokens) * sizeof(float);
  dim3 grid(num_requests, H);
#define IFX_SCAN(R, TO)                                                                                          \
  do {                                                                                                           \
    auto kern = wkv_scan_kernel<R, TO>;                                                                          \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    kern<<<grid, threads, smem, stream>>>(r, k, v, w_raw, g, w0, u, norm_w, eps, s_state, prev_state, slot_stride, \
                                          x, C, cu_seqlens, req_slot, o_scratch, (TO*)y, H, D, ks);              \
  } while (0)
  if (out_dtype == IFX_DT_F32) {
    if (rmax == 16) IFX_SCAN(16, float); else IFX_SCAN(64, float);
  } else if (out_dtype == IFX_DT_BF16) {
    if (rmax == 16) IFX_SCAN(16, __nv_bfloat16); else IFX_SCAN(64, __nv_bfloat16);
  } else {
    return IFX_E_DTYPE;
  }
#undef IFX_SCAN
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
