// Kernels of layers that norm a sublayer's output before it joins the residual
// stream, and the small element kernels such layers bring with them.
//
//   postnorm_add_rmsnorm   x += y / rms(y) * w_post           (x float32, in place)
//                          h  = x / rms(x) * w_next           (optional second stage)
//                          h  = x in the output's dtype       (out given, w_next null: the next sublayer reads x itself)
//                          y may arrive as the float32 partial sums [splits, rows, hidden] of a K-split product
//   concat_cast            out[t] = [a[t]; b[t]] in the run's dtype, a and b float32
//   xielu                  z -> a_pos z^2 + z/2 (z > 0), a_neg (e^z - 1 - z) + z/2 (z <= 0)
//   softcap                v -> cap tanh(v / cap), float32 in place
//
// Norms reduce in float32 with a block reduction of fixed order, one block per row:
// a row's result does not depend on which other rows share the launch.
#include "common.cuh"

namespace ifx {

// What a row that is its request's only token in the step needs for the short convolution behind the norm
// (see short_conv.cu): its taps, and the request's state, which the row reads and moves on itself.
struct SingleTokenConv {
  const float* w;            // [hidden, taps], null: no convolution
  float* state;              // this convolution's [taps - 1, hidden] of slot 0
  long long slot_stride;     // floats from one slot to the next
  const int* token_req;
  const int* req_slot;
  int taps;
};

// Few rows make this kernel a chain of round trips to memory, not a stream: everything a thread will need
// that does not depend on a reduction (its first elements of x and of the norm weights) is asked for before
// the first reduction, the slices of a K-split product are loaded in batches before they are added, and a
// row gets 1,024 threads when there are few rows.
template <typename TY, typename TO>
__global__ void __launch_bounds__(1024) postnorm_add_rmsnorm_kernel(
    float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ w_post, float eps_post,
    const float* __restrict__ w_next, float eps_next, TO* __restrict__ out, int hidden, int splits,
    size_t split_stride, SingleTokenConv conv) {
  extern __shared__ float row_s[];                       // the row, kept between the passes
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  float* xr = x + row * hidden;
  const TY* yr = y + row * hidden;
  constexpr int PRE = 2;                                 // elements per thread fetched ahead
  float x_pre[PRE], wp_pre[PRE], wn_pre[PRE];
#pragma unroll
  for (int j = 0; j < PRE; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    x_pre[j] = i < hidden ? xr[i] : 0.0f;
    wp_pre[j] = i < hidden ? w_post[i] : 0.0f;
    wn_pre[j] = (i < hidden && out != nullptr && w_next != nullptr) ? w_next[i] : 0.0f;
  }
  // the convolution's taps and the request's state do not depend on a reduction either (up to 4 taps: 3 cells)
  const bool conv_pre = conv.w != nullptr && conv.taps <= 4;
  float* st_pre = nullptr;
  float old_pre[PRE][3], tap_pre[PRE][4];
  if (conv_pre) {
    st_pre = conv.taps > 1 ? conv.state + (long long)conv.req_slot[conv.token_req[row]] * conv.slot_stride : nullptr;
#pragma unroll
    for (int j = 0; j < PRE; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
#pragma unroll
      for (int k = 0; k < 3; ++k)                          // old_pre[j][k]: the input k + 1 steps back
        old_pre[j][k] = (i < hidden && k < conv.taps - 1) ? st_pre[(size_t)(conv.taps - 2 - k) * hidden + i] : 0.0f;
#pragma unroll
      for (int k = 0; k < 4; ++k)                          // tap_pre[j][k]: the tap of the input k steps back
        tap_pre[j][k] = (i < hidden && k < conv.taps) ? conv.w[(size_t)i * conv.taps + conv.taps - 1 - k] : 0.0f;
    }
  }
  float ss = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_f32(yr[i]);
    int s = 1;
    for (; s + 4 <= splits; s += 4) {                    // K-split partial sums: four loads in flight, added in split order
      const float p0 = to_f32(yr[(size_t)s * split_stride + i]), p1 = to_f32(yr[(size_t)(s + 1) * split_stride + i]);
      const float p2 = to_f32(yr[(size_t)(s + 2) * split_stride + i]), p3 = to_f32(yr[(size_t)(s + 3) * split_stride + i]);
      v += p0; v += p1; v += p2; v += p3;
    }
    for (; s < splits; ++s) v += to_f32(yr[(size_t)s * split_stride + i]);
    row_s[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float r1 = rsqrtf(ss / (float)hidden + eps_post);
  float ss2 = 0.0f;
  auto add_row = [&](int i, float xi, float wi) {
    const float v = xi + row_s[i] * r1 * wi;
    xr[i] = v;
    row_s[i] = v;
    ss2 = fmaf(v, v, ss2);
  };
#pragma unroll
  for (int j = 0; j < PRE; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < hidden) add_row(i, x_pre[j], wp_pre[j]);
  }
  for (int i = threadIdx.x + PRE * blockDim.x; i < hidden; i += blockDim.x) add_row(i, xr[i], w_post[i]);
  if (out == nullptr) return;
  TO* o = out + row * hidden;
  if (w_next == nullptr) {                               // no second norm: the updated row in the output's dtype
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<TO>(row_s[i]);
    return;
  }
  ss2 = block_sum(ss2, scratch);
  const float r2 = rsqrtf(ss2 / (float)hidden + eps_next);
  if (conv.w == nullptr) {
#pragma unroll
    for (int j = 0; j < PRE; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < hidden) o[i] = from_f32<TO>(row_s[i] * r2 * wn_pre[j]);
    }
    for (int i = threadIdx.x + PRE * blockDim.x; i < hidden; i += blockDim.x) o[i] = from_f32<TO>(row_s[i] * r2 * w_next[i]);
    return;
  }
  // h + conv(h) for a single token: the inputs before it are the state; afterwards the state ends with h
  float* st = conv.state + (long long)conv.req_slot[conv.token_req[row]] * conv.slot_stride;
  const int taps = conv.taps;
  auto conv_one = [&](int i, float wn) {
    const float* wc = conv.w + (size_t)i * taps;
    float old[15], wk[15];                                               // the input k + 1 steps back, and its tap
#pragma unroll
    for (int k = 0; k < 15; ++k) {
      old[k] = k < taps - 1 ? st[(size_t)(taps - 2 - k) * hidden + i] : 0.0f;
      wk[k] = k < taps - 1 ? wc[taps - 2 - k] : 0.0f;
    }
    const float h = to_f32(from_f32<TO>(row_s[i] * r2 * wn));            // the convolution reads h in the run's dtype
    float acc = fmaf(wc[taps - 1], h, h);
#pragma unroll
    for (int k = 0; k < 15; ++k)
      if (k < taps - 1) {
        acc = fmaf(wk[k], old[k], acc);
        st[(size_t)(taps - 2 - k) * hidden + i] = k == 0 ? h : old[k - 1];
      }
    o[i] = from_f32<TO>(acc);
  };
#pragma unroll
  for (int j = 0; j < PRE; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i >= hidden) continue;
    if (!conv_pre) {
      conv_one(i, wn_pre[j]);
      continue;
    }
    // the same sums in the same order, from what was fetched at the start
    const float h = to_f32(from_f32<TO>(row_s[i] * r2 * wn_pre[j]));
    float acc = fmaf(tap_pre[j][0], h, h);
#pragma unroll
    for (int k = 0; k < 3; ++k)
      if (k < taps - 1) {
        acc = fmaf(tap_pre[j][k + 1], old_pre[j][k], acc);
        st_pre[(size_t)(taps - 2 - k) * hidden + i] = k == 0 ? h : old_pre[j][k - 1 < 0 ? 0 : k - 1];
      }
    o[i] = from_f32<TO>(acc);
  }
  for (int i = threadIdx.x + PRE * blockDim.x; i < hidden; i += blockDim.x) conv_one(i, w_next[i]);
}

// Many rows: the same three passes with four elements per thread and step (16-byte loads of x, the weights and the
// row buffer, 8 or 16 of y), for widths that are multiples of 4.  No convolution here: that is for steps of single tokens.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TY, typename TO>
__global__ void __launch_bounds__(256) postnorm_add_rmsnorm_rows_kernel(
    float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ w_post, float eps_post,
    const float* __restrict__ w_next, float eps_next, TO* __restrict__ out, int hidden, int splits,
    size_t split_stride) {
  extern __shared__ __align__(16) float row_s[];
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  float* xr = x + row * hidden;
  const TY* yr = y + row * hidden;
  const int step = blockDim.x * 4;
  float ss = 0.0f;
  for (int i = threadIdx.x * 4; i < hidden; i += step) {
    float4 v = ld4(yr + i);
    for (int s = 1; s < splits; ++s) {
      const float4 p = ld4(yr + (size_t)s * split_stride + i);
      v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
    }
    st4(row_s + i, v);
    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
  }
  ss = block_sum(ss, scratch);
  const float r1 = rsqrtf(ss / (float)hidden + eps_post);
  float ss2 = 0.0f;
  for (int i = threadIdx.x * 4; i < hidden; i += step) {
    const float4 xv = ld4(xr + i), wv = ld4(w_post + i), yv = ld4(row_s + i);
    const float4 v = make_float4(xv.x + yv.x * r1 * wv.x, xv.y + yv.y * r1 * wv.y, xv.z + yv.z * r1 * wv.z,
                                 xv.w + yv.w * r1 * wv.w);
    st4(xr + i, v);
    st4(row_s + i, v);
    ss2 = fmaf(v.x, v.x, ss2); ss2 = fmaf(v.y, v.y, ss2); ss2 = fmaf(v.z, v.z, ss2); ss2 = fmaf(v.w, v.w, ss2);
  }
  if (out == nullptr) return;
  TO* o = out + row * hidden;
  if (w_next == nullptr) {
    for (int i = threadIdx.x * 4; i < hidden; i += step) st4(o + i, ld4(row_s + i));
    return;
  }
  ss2 = block_sum(ss2, scratch);
  const float r2 = rsqrtf(ss2 / (float)hidden + eps_next);
  for (int i = threadIdx.x * 4; i < hidden; i += step) {
    const float4 v = ld4(row_s + i), wv = ld4(w_next + i);
    st4(o + i, make_float4(v.x * r2 * wv.x, v.y * r2 * wv.y, v.z * r2 * wv.z, v.w * r2 * wv.w));
  }
}

template <typename T>
__global__ void concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out,
                                   long long rows, int hidden) {
  const long long n = rows * 2 * hidden;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / (2 * hidden);
    const int c = (int)(i % (2 * hidden));
    out[i] = from_f32<T>(c < hidden ? a[t * hidden + c] : b[t * hidden + c - hidden]);
  }
}

__device__ __forceinline__ float xielu_f(float z, float a_pos, float a_neg) {
  return z > 0.0f ? fmaf(a_pos * z, z, 0.5f * z) : fmaf(a_neg, expm1f(z) - z, 0.5f * z);
}

// splits > 1: z is float32 [splits, n], the partial sums of a K-split product, added in split order first.
template <typename TI, typename TO>
__global__ void xielu_kernel(const TI* __restrict__ z, TO* __restrict__ out, long long n, float a_pos, float a_neg,
                             int splits) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = to_f32(z[i]);
    for (int s = 1; s < splits; ++s) v += to_f32(z[(long long)s * n + i]);
    out[i] = from_f32<TO>(xielu_f(v, a_pos, a_neg));
  }
}

// e^z - 1 through the fast exponential: its error of a few 1e-7 is far below what rounding the result to bfloat16 does
// (the result is dominated by z / 2 where e^z - 1 - z is small).
__device__ __forceinline__ float xielu_fast(float z, float a_pos, float a_neg) {
  return z > 0.0f ? fmaf(a_pos * z, z, 0.5f * z) : fmaf(a_neg, (__expf(z) - 1.0f) - z, 0.5f * z);
}

// The same, eight bfloat16 (16 bytes) per thread and step, for element counts that are multiples of 8.
__global__ void xielu_bf16x8_kernel(const __nv_bfloat16* __restrict__ z, __nv_bfloat16* __restrict__ out, long long n8,
                                    float a_pos, float a_neg) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 raw = reinterpret_cast<const uint4*>(z)[i];
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h2[k]);
      h2[k] = __floats2bfloat162_rn(xielu_fast(f.x, a_pos, a_neg), xielu_fast(f.y, a_pos, a_neg));
    }
    reinterpret_cast<uint4*>(out)[i] = raw;
  }
}

__global__ void softcap_kernel(float* __restrict__ v, long long n, float cap) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    v[i] = cap * tanhf(v[i] / cap);
}

inline unsigned grid_for(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  return (unsigned)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace ifx

using namespace ifx;

extern "C" {

// y_dtype: dtype of y; out_dtype: dtype of out (ignored when out is null: first stage only).
// splits > 1: y is float32 [splits, T, hidden].
// conv_w non-null (only for steps in which every request brings one token, and with `out`): the rows leave as
// h + conv(h), with `conv_state` (this convolution's part of slot 0, slots conv_slot_stride floats apart) read and moved on.
int ifx_postnorm_add_rmsnorm(float* x, const void* y, const float* w_post, float eps_post, const float* w_next,
                             float eps_next, void* out, int T, int hidden, int y_dtype, int out_dtype, int splits,
                             const float* conv_w, int taps, float* conv_state, long long conv_slot_stride,
                             const int* token_req, const int* req_slot, cudaStream_t stream) {
  if (T <= 0) return 0;
  SingleTokenConv conv = {conv_w, conv_state, conv_slot_stride, token_req, req_slot, taps};
  if (conv_w != nullptr && (out == nullptr || taps < 1 || taps > 16 || (taps > 1 && conv_state == nullptr) ||
                            token_req == nullptr || req_slot == nullptr))
    return IFX_E_BADARG;
  if (hidden <= 0 || splits < 1 || (splits > 1 && y_dtype != IFX_DT_F32)) return IFX_E_BADARG;
  const size_t split_stride = (size_t)T * hidden;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return IFX_E_TOOBIG;
  // A float32 run (float32 in, float32 out, no slices) always takes the same kernel with the same block, so that a
  // row's sums are added in an order that depends on the width alone, never on how many rows share the launch.
  const bool exact = y_dtype == IFX_DT_F32 && splits == 1 && (out == nullptr || out_dtype == IFX_DT_F32);
  const int threads = (!exact && T <= 512 && hidden > 512) ? 1024 : 256;  // few rows: more threads a row
  const bool rows_path = !exact && T > 512 && conv_w == nullptr && hidden % 4 == 0 && (uintptr_t)x % 16 == 0 &&
                         (uintptr_t)y % 16 == 0 && (out == nullptr || (uintptr_t)out % 16 == 0) &&
                         (uintptr_t)w_post % 16 == 0 && (w_next == nullptr || (uintptr_t)w_next % 16 == 0);
  if (conv_w != nullptr && w_next == nullptr) return IFX_E_BADARG;
#define IFX_LAUNCH(TY, TO)                                                                                         \
  do {                                                                                                             \
    if (rows_path) {                                                                                               \
      auto kern = postnorm_add_rmsnorm_rows_kernel<TY, TO>;                                                        \
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
      kern<<<T, 256, smem, stream>>>(x, (const TY*)y, w_post, eps_post, w_next, eps_next, (TO*)out, hidden, splits, \
                                     split_stride);                                                                \
    } else {                                                                                                       \
      auto kern = postnorm_add_rmsnorm_kernel<TY, TO>;                                                             \
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
      kern<<<T, threads, smem, stream>>>(x, (const TY*)y, w_post, eps_post, w_next, eps_next, (TO*)out, hidden,    \
                                         splits, split_stride, conv);                                              \
    }                                                                                                              \
  } while (0)
  const int od = out == nullptr ? IFX_DT_F32 : out_dtype;
  if (y_dtype == IFX_DT_F32 && od == IFX_DT_F32) IFX_LAUNCH(float, float);
  else if (y_dtype == IFX_DT_BF16 && od == IFX_DT_BF16) IFX_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (y_dtype == IFX_DT_F32 && od == IFX_DT_BF16) IFX_LAUNCH(float, __nv_bfloat16);
  else if (y_dtype == IFX_DT_BF16 && od == IFX_DT_F32) IFX_LAUNCH(__nv_bfloat16, float);
  else return IFX_E_DTYPE;
#undef IFX_LAUNCH
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_concat_cast(const float* a, const float* b, void* out, int T, int hidden, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hidden <= 0) return IFX_E_BADARG;
  const long long n = (long long)T * 2 * hidden;
  if (dtype == IFX_DT_F32) concat_cast_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>(a, b, (float*)out, T, hidden);
  else if (dtype == IFX_DT_BF16)
    concat_cast_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, stream>>>(a, b, (__nv_bfloat16*)out, T, hidden);
  else return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_xielu(const void* z, void* out, long long n, float a_pos, float a_neg, int in_dtype, int out_dtype, int splits,
              cudaStream_t stream) {
  if (n <= 0) return 0;
  if (splits < 1 || (splits > 1 && in_dtype != IFX_DT_F32)) return IFX_E_BADARG;
  if (in_dtype == IFX_DT_F32 && out_dtype == IFX_DT_F32)
    xielu_kernel<float, float><<<grid_for(n, 256), 256, 0, stream>>>((const float*)z, (float*)out, n, a_pos, a_neg, splits);
  else if (in_dtype == IFX_DT_BF16 && out_dtype == IFX_DT_BF16 && n % 8 == 0 && (uintptr_t)z % 16 == 0 &&
           (uintptr_t)out % 16 == 0)
    xielu_bf16x8_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)z, (__nv_bfloat16*)out, n / 8,
                                                                  a_pos, a_neg);
  else if (in_dtype == IFX_DT_BF16 && out_dtype == IFX_DT_BF16)
    xielu_kernel<__nv_bfloat16, __nv_bfloat16><<<grid_for(n, 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)z, (__nv_bfloat16*)out, n, a_pos, a_neg, splits);
  else if (in_dtype == IFX_DT_F32 && out_dtype == IFX_DT_BF16)
    xielu_kernel<float, __nv_bfloat16><<<grid_for(n, 256), 256, 0, stream>>>((const float*)z, (__nv_bfloat16*)out, n,
                                                                             a_pos, a_neg, splits);
  else return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_softcap(float* v, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!(cap > 0.0f)) return IFX_E_BADARG;
  softcap_kernel<<<grid_for(n, 256), 256, 0, stream>>>(v, n, cap);
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
