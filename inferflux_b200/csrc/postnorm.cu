// Kernels of layers that norm a sublayer's output before it joins the residual
// stream, and the small element kernels such layers bring with them.
//
//   postnorm_add_rmsnorm   x += y / rms(y) * w_post           (x float32, in place)
//                          h  = x / rms(x) * w_next           (optional second stage)
//   concat_cast            out[t] = [a[t]; b[t]] in the run's dtype, a and b float32
//   xielu                  z -> a_pos z^2 + z/2 (z > 0), a_neg (e^z - 1 - z) + z/2 (z <= 0)
//   softcap                v -> cap tanh(v / cap), float32 in place
//
// Norms reduce in float32 with a block reduction of fixed order, one block per row:
// a row's result does not depend on which other rows share the launch.
#include "common.cuh"

namespace ifx {

template <typename TY, typename TO>
__global__ void __launch_bounds__(256) postnorm_add_rmsnorm_kernel(
    float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ w_post, float eps_post,
    const float* __restrict__ w_next, float eps_next, TO* __restrict__ out, int hidden) {
  extern __shared__ float row_s[];                       // the row, kept between the passes
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  float* xr = x + row * hidden;
  const TY* yr = y + row * hidden;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = to_f32(yr[i]);
    row_s[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float r1 = rsqrtf(ss / (float)hidden + eps_post);
  float ss2 = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = xr[i] + row_s[i] * r1 * w_post[i];
    xr[i] = v;
    row_s[i] = v;
    ss2 = fmaf(v, v, ss2);
  }
  if (out == nullptr) return;
  ss2 = block_sum(ss2, scratch);
  const float r2 = rsqrtf(ss2 / (float)hidden + eps_next);
  TO* o = out + row * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<TO>(row_s[i] * r2 * w_next[i]);
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

template <typename T>
__global__ void xielu_kernel(const T* __restrict__ z, T* __restrict__ out, long long n, float a_pos, float a_neg) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(xielu_f(to_f32(z[i]), a_pos, a_neg));
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
int ifx_postnorm_add_rmsnorm(float* x, const void* y, const float* w_post, float eps_post, const float* w_next,
                             float eps_next, void* out, int T, int hidden, int y_dtype, int out_dtype,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hidden <= 0) return IFX_E_BADARG;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return IFX_E_TOOBIG;
  if (out != nullptr && w_next == nullptr) return IFX_E_BADARG;
#define IFX_LAUNCH(TY, TO)                                                                                         \
  do {                                                                                                             \
    auto kern = postnorm_add_rmsnorm_kernel<TY, TO>;                                                               \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    kern<<<T, 256, smem, stream>>>(x, (const TY*)y, w_post, eps_post, w_next, eps_next, (TO*)out, hidden);         \
  } while (0)
  const int od = out == nullptr ? y_dtype : out_dtype;
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

int ifx_xielu(const void* z, void* out, long long n, float a_pos, float a_neg, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dtype == IFX_DT_F32)
    xielu_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((const float*)z, (float*)out, n, a_pos, a_neg);
  else if (dtype == IFX_DT_BF16)
    xielu_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, stream>>>((const __nv_bfloat16*)z, (__nv_bfloat16*)out, n,
                                                                      a_pos, a_neg);
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
