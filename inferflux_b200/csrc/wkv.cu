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
// Layout of a thread block of the scan: thread (j, s) owns value channel j and four (for the largest heads eight)
// key channels i = s, s + KS, s + 2 KS, ... of S in registers (KS a power of two up to 32 that depends on the
// head size alone; the KS threads of a channel are neighbours in a warp and add their shares by shuffles).  r, k, w and v of up to 32 tokens arrive in shared
// memory at a time, so the block synchronises three times per 32 tokens, not per token.
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

constexpr int kScanThreads = 1024;   // the most threads a block of the scan has

__device__ __forceinline__ void cp_async_4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// out / rms(out) * norm_w * silu(g) for one (token, head), by one warp: the same code whether the scan's block or
// the kernel of its own runs it, so that both give the same bits.
template <typename TO>
__device__ __forceinline__ void wkv_head_norm(const float* __restrict__ o, const float* __restrict__ g,
                                              const float* __restrict__ norm_w, float eps, TO* __restrict__ y, int D,
                                              int lane) {
  float ss = 0.0f;
  for (int i = lane; i < D; i += 32) ss = fmaf(o[i], o[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)D + eps);
  for (int i = lane; i < D; i += 32) {
    const float gate = g[i];
    y[i] = from_f32<TO>(o[i] * inv * norm_w[i] * (gate / (1.0f + expf(-gate))));
  }
}

// grid (requests, heads, column groups): a block owns `DC` value channels of one head of one request.  A column of S
// depends on no other column, so the split changes no sum.  Inputs of `TB` tokens at a time arrive by cp.async in
// one of two buffers while the tokens of the other are worked on.  With one column group the block norms its own
// outputs at the end (`fused_norm`); otherwise wkv_norm_kernel does.
template <int KS, int R, typename TO>
__global__ void __launch_bounds__(kScanThreads) wkv_scan_kernel(
    const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
    const float* __restrict__ w_raw, const float* __restrict__ g, const float* __restrict__ w0,
    const float* __restrict__ u, const float* __restrict__ norm_w, float eps, float* __restrict__ s_state,
    float* __restrict__ prev_state, long long slot_stride, const float* __restrict__ x, int C,
    const int* __restrict__ cu_seqlens, const int* __restrict__ req_slot, float* __restrict__ o_scratch,
    TO* __restrict__ y, int H, int D, int DC, int TB, int fused_norm, int wide_copies, int ld, int ld_w) {
  extern __shared__ __align__(16) float smem[];
  constexpr int DP = KS * R;                         // a staged row of r, k or w: D numbers, then zeros up to KS * R
  const int per_buf = TB * (3 * DP + DC);
  float* b_s = smem + 2 * per_buf;                   // [TB] bonus sums of the chunk at work
  const int req = blockIdx.x, head = blockIdx.y, j0 = blockIdx.z * DC;
  const int cols = min(DC, D - j0);                  // value channels of this block
  const int lo = cu_seqlens[req], hi = cu_seqlens[req + 1];
  const int slot = req_slot[req];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int jl = tid / KS, s = tid % KS;
  const bool active = jl < cols;
  const int j = j0 + jl;
  const int HD = H * D;
  float* S_g = s_state + (long long)slot * slot_stride + (size_t)head * D * D;
  float S[R];
#pragma unroll
  for (int m = 0; m < R; ++m) {
    const int i = s + KS * m;
    S[m] = (active && i < D) ? S_g[(size_t)i * D + j] : 0.0f;
  }
  // what lies behind a row's D numbers stays zero for good: a key channel that does not exist adds nothing
  for (int idx = tid; idx < 2 * per_buf + TB; idx += blockDim.x) smem[idx] = 0.0f;
  __syncthreads();
  auto fetch = [&](int t0, int buf) {                // tokens [t0, t0 + TB) of the span into buffer `buf`
    const int nt = min(TB, hi - t0);
    float* r_s = smem + buf * per_buf;
    float* k_s = r_s + TB * DP;
    float* w_s = k_s + TB * DP;
    float* v_s = w_s + TB * DP;
    if (wide_copies) {
      const int d4 = D >> 2, c4 = cols >> 2;
      for (int idx = tid; idx < nt * d4; idx += blockDim.x) {
        const int tt = idx / d4, i = (idx % d4) * 4;
        const size_t src = (size_t)(t0 + tt) * ld + (size_t)head * D + i;
        cp_async_16(r_s + tt * DP + i, r + src);
        cp_async_16(k_s + tt * DP + i, k + src);
        cp_async_16(w_s + tt * DP + i, w_raw + (size_t)(t0 + tt) * ld_w + (size_t)head * D + i);
      }
      for (int idx = tid; idx < nt * c4; idx += blockDim.x) {
        const int tt = idx / c4, i = (idx % c4) * 4;
        cp_async_16(v_s + tt * DC + i, v + (size_t)(t0 + tt) * ld + (size_t)head * D + j0 + i);
      }
    } else {
      for (int idx = tid; idx < nt * D; idx += blockDim.x) {
        const int tt = idx / D, i = idx % D;
        const size_t src = (size_t)(t0 + tt) * ld + (size_t)head * D + i;
        cp_async_4(r_s + tt * DP + i, r + src);
        cp_async_4(k_s + tt * DP + i, k + src);
        cp_async_4(w_s + tt * DP + i, w_raw + (size_t)(t0 + tt) * ld_w + (size_t)head * D + i);
      }
      for (int idx = tid; idx < nt * cols; idx += blockDim.x) {
        const int tt = idx / cols, i = idx % cols;
        cp_async_4(v_s + tt * DC + i, v + (size_t)(t0 + tt) * ld + (size_t)head * D + j0 + i);
      }
    }
  };
  if (lo < hi) fetch(lo, 0);
  cp_async_commit();
  int buf = 0;
  for (int t0 = lo; t0 < hi; t0 += TB, buf ^= 1) {
    const int nt = min(TB, hi - t0);
    if (t0 + TB < hi) fetch(t0 + TB, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();                              // everything but the copies just asked for has landed
    __syncthreads();
    float* r_s = smem + buf * per_buf;
    float* k_s = r_s + TB * DP;
    float* w_s = k_s + TB * DP;
    float* v_s = w_s + TB * DP;
    for (int idx = tid; idx < nt * D; idx += blockDim.x) {        // the decay, where the exponent was copied to
      const int tt = idx / D, i = idx % D;
      w_s[tt * DP + i] = expf(-expf(w_s[tt * DP + i] + w0[head * D + i]));
    }
    for (int tt = warp; tt < nt; tt += nwarps) {                   // the bonus of the present token: one number per token
      float b = 0.0f;
      for (int i = lane; i < D; i += 32) b = fmaf(r_s[tt * DP + i] * u[head * D + i], k_s[tt * DP + i], b);
      b = warp_sum(b);
      if (lane == 0) b_s[tt] = b;
    }
    __syncthreads();
#pragma unroll 4
    for (int tt = 0; tt < nt; ++tt) {
      const float* rr = r_s + tt * DP + s;
      const float* kk = k_s + tt * DP + s;
      const float* ww = w_s + tt * DP + s;
      const float vj = active ? v_s[tt * DC + jl] : 0.0f;
      float acc = 0.0f;
#pragma unroll
      for (int m = 0; m < R; ++m) {
        acc = fmaf(rr[KS * m], S[m], acc);
        S[m] = fmaf(ww[KS * m], S[m], kk[KS * m] * vj);
      }
#pragma unroll
      for (int o = 1; o < KS; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (active && s == 0) o_scratch[(size_t)(t0 + tt) * HD + (size_t)head * D + j] = fmaf(b_s[tt], vj, acc);
    }
    __syncthreads();                                 // the buffer is free for the copies of the chunk after next
  }
  cp_async_wait<0>();
#pragma unroll
  for (int m = 0; m < R; ++m) {
    const int i = s + KS * m;
    if (active && i < D) S_g[(size_t)i * D + j] = S[m];
  }
  if (head == 0 && blockIdx.z == 0 && hi > lo) {       // the step's last input is the next step's "token before"
    float* p = prev_state + (long long)slot * slot_stride;
    const float* last = x + (size_t)(hi - 1) * C;
    for (int i = tid; i < C; i += blockDim.x) p[i] = last[i];
  }
  if (!fused_norm) return;
  // the block's own writes to o_scratch are visible to it after the barrier at the end of the loop
  for (int t = lo + warp; t < hi; t += nwarps) {
    const size_t base = (size_t)t * HD + (size_t)head * D;
    wkv_head_norm<TO>(o_scratch + base, g + (size_t)t * ld + (size_t)head * D, norm_w + head * D, eps, y + base, D, lane);
  }
}

template <typename TO>
__global__ void wkv_norm_kernel(const float* __restrict__ o, const float* __restrict__ g, const float* __restrict__ norm_w,
                                float eps, TO* __restrict__ y, long long items, int H, int D, int ld) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const int head = (int)(item % H);
  const size_t base = (size_t)item * D;              // item = token * H + head
  wkv_head_norm<TO>(o + base, g + (size_t)(item / H) * ld + (size_t)head * D, norm_w + head * D, eps, y + base, D,
                    threadIdx.x & 31);
}

}  // namespace ifx

using namespace ifx;

extern "C" {

int ifx_token_shift_mix(const float* x, const float* mu, const float* prev_state, long long slot_stride,
                        const int* token_req, const int* req_slot, const int* cu_seqlens, void* out, int T, int C,
                        int n_mix, int out_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C <= 0 || n_mix <= 0 || prev_state == nullptr) return IFX_E_BADARG;
  const int threads = T <= 64 ? (C >= 2048 ? 1024 : (C >= 512 ? 512 : 128)) : (C >= 1024 ? 256 : (C >= 256 ? 128 : 64));
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

// r, k, v, w_raw, g: float32 [T, H * D] in rows `ld` floats apart (`ld_w` for w_raw): they may be column
// blocks of one wider matrix.  s_state / prev_state: slot 0's matrix block [H, D, D] and input row [C]
// inside the state tensor, slots slot_stride floats apart.  o_scratch: float32 [T, H * D].  y: [T, H * D].
int ifx_wkv_scan(const float* r, const float* k, const float* v, const float* w_raw, const float* g, const float* w0,
                 const float* u, const float* norm_w, float eps, float* s_state, float* prev_state,
                 long long slot_stride, const float* x, int C, const int* cu_seqlens, const int* req_slot,
                 float* o_scratch, void* y, int num_requests, int num_tokens, int H, int D, int ld, int ld_w, int out_dtype,
                 cudaStream_t stream) {
  if (num_requests <= 0 || num_tokens <= 0) return 0;
  if (H <= 0 || D <= 0 || D > 256 || H > 65535 || ld < H * D || ld_w < H * D) return IFX_E_BADARG;
  // threads per value channel (a power of two that depends on the head size alone, so that a sum's order does too)
  // and key channels per thread: four, eight for the largest heads
  int ks = 1;
  while (ks < 32 && ks * 4 < D) ks *= 2;
  int rows = ks * 4 >= D ? 4 : 8;
  const int longest = num_tokens - (num_requests - 1);                 // no span is longer than this
  // A bfloat16 run's long spans (prompt portions) are bound by the latency of one warp's instructions per token:
  // two key channels a thread make twice the warps with half the work each.  The float32 run keeps one split per
  // head size, so that its sums have one order however the tokens are cut.
  // (measured on one prompt of 2,048 tokens: 24 heads of 64 channels 631 -> 530 us, but 56 heads 631 -> 727 us: with
  // enough threads to fill the SMs the extra shuffles only cost)
  if (out_dtype == IFX_DT_BF16 && longest >= 64 && rows == 4 && ks <= 16 && ks * 4 == D && D >= 16 &&
      (long long)num_requests * H * D * ks < 40000) {
    ks *= 2;
    rows = 2;
  }
  const int dp = ks * rows;
  // value channels per block: as many as a block holds; fewer while the grid does not fill the SMs
  int dc = D;
  while (dc * ks > kScanThreads) dc = (dc + 1) / 2;
  while ((long long)num_requests * H * ((D + dc - 1) / dc) < 148 && dc * ks > 64 && dc % 8 == 0) dc /= 2;
  const int groups = (D + dc - 1) / dc;
  const int threads = (dc * ks + 31) / 32 * 32;
  int tb = longest < 32 ? (longest < 16 ? 16 : longest) : (longest >= 128 ? 64 : 32);
  while (tb > 4 && ((size_t)2 * tb * (3 * dp + dc) + tb) * sizeof(float) > 160 * 1024) tb /= 2;
  const size_t smem = ((size_t)2 * tb * (3 * dp + dc) + tb) * sizeof(float);
  const int wide = (D % 4 == 0 && dc % 4 == 0 && ld % 4 == 0 && ld_w % 4 == 0 && ((uintptr_t)r | (uintptr_t)k | (uintptr_t)v | (uintptr_t)w_raw) % 16 == 0) ? 1 : 0;
  const int fused = groups == 1 ? 1 : 0;
  dim3 grid(num_requests, H, groups);
#define IFX_SCAN(KS_, R_, TO)                                                                                    \
  do {                                                                                                           \
    auto kern = wkv_scan_kernel<KS_, R_, TO>;                                                                    \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    kern<<<grid, threads, smem, stream>>>(r, k, v, w_raw, g, w0, u, norm_w, eps, s_state, prev_state, slot_stride, \
                                          x, C, cu_seqlens, req_slot, o_scratch, (TO*)y, H, D, dc, tb, fused, wide, ld, ld_w); \
    if (!fused) {                                                                                                \
      const long long items = (long long)num_tokens * H;                                                        \
      wkv_norm_kernel<TO><<<(unsigned)((items + 7) / 8), 256, 0, stream>>>(o_scratch, g, norm_w, eps, (TO*)y, items, H, D, ld); \
    }                                                                                                            \
  } while (0)
#define IFX_SCAN_KS(TO)                                   \
  do {                                                    \
    if (rows == 2 && ks == 8) IFX_SCAN(8, 2, TO);         \
    else if (rows == 2 && ks == 16) IFX_SCAN(16, 2, TO);  \
    else if (rows == 2) IFX_SCAN(32, 2, TO);              \
    else if (rows == 8) IFX_SCAN(32, 8, TO);              \
    else if (ks == 1) IFX_SCAN(1, 4, TO);                 \
    else if (ks == 2) IFX_SCAN(2, 4, TO);                 \
    else if (ks == 4) IFX_SCAN(4, 4, TO);                 \
    else if (ks == 8) IFX_SCAN(8, 4, TO);                 \
    else if (ks == 16) IFX_SCAN(16, 4, TO);               \
    else IFX_SCAN(32, 4, TO);                             \
  } while (0)
  if (out_dtype == IFX_DT_F32) IFX_SCAN_KS(float);
  else if (out_dtype == IFX_DT_BF16) IFX_SCAN_KS(__nv_bfloat16);
  else return IFX_E_DTYPE;
#undef IFX_SCAN_KS
#undef IFX_SCAN
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
