// Dynamic tanh (a norm without mean or variance: tanh(alpha x) w + b, alpha a scalar) fused with the
// residual sum around it.  One pass does, per element,
//
//     r  = residual (or 0 where the stream starts here)
//     r += mult * post(y)        post = a dynamic tanh (the norm behind a sublayer), or the identity
//     r += add[c]                a vector of the row's width, where one is given
//     residual = r               (32-bit, in place or into a stream of its own)
//     out = pre(r)               pre = a dynamic tanh (the norm in front of the next sublayer), or the identity
//
// so that the norm behind a sublayer, the scaled sum into the stream and the norm in front of the next
// sublayer cost one launch.  Everything is 32-bit (accurate tanhf); y and out have their own types, and
// out's rows may be a slice of a wider buffer.
#include <math.h>
#include "common.cuh"

namespace {
template <typename TY, typename TO>
__global__ void dyt_step_kernel(const TY* y, long long y_stride, float post_alpha, const float* __restrict__ post_w,
                                const float* __restrict__ post_b, float mult, const float* __restrict__ add,
                                const float* res_in, float* res_out, float pre_alpha, const float* __restrict__ pre_w,
                                const float* __restrict__ pre_b, TO* out, long long out_stride, long long rows, int cols) {
  pdl_wait();
  pdl_trigger();
  const long long n = rows * cols;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / cols;
    const int c = (int)(idx - r * cols);
    float s = res_in != nullptr ? res_in[idx] : 0.f;
    if (y != nullptr) {
      float v = to_f(y[r * y_stride + c]);
      if (post_w != nullptr) v = fmaf(tanhf(post_alpha * v), post_w[c], post_b[c]);
      s = fmaf(mult, v, s);
    }
    if (add != nullptr) s += add[c];
    if (res_out != nullptr) res_out[idx] = s;
    if (out != nullptr) {
      const float o = pre_w != nullptr ? fmaf(tanhf(pre_alpha * s), pre_w[c], pre_b[c]) : s;
      out[r * out_stride + c] = from_f<TO>(o);
    }
  }
}
}  // namespace

// y (of y_dtype, rows of y_stride) may be null; post_w / post_b null: y is added as it is; add null: nothing
// more is added; res_in null: the stream starts at zero; res_out null: the stream is not written (res_in and
// res_out may be the same array); pre_w / pre_b null: out = the stream; out null: nothing is written there.
FMX_EXPORT int fmx_dyt_step(const void* y, long long y_stride, int y_dtype, float post_alpha, const float* post_w,
                            const float* post_b, float mult, const float* add, const float* res_in, float* res_out,
                            float pre_alpha, const float* pre_w, const float* pre_b, void* out, long long out_stride,
                            int out_dtype, int rows, int cols, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  if (rows < 0 || cols < 0 || (y != nullptr && y_stride < cols) || (out != nullptr && out_stride < cols))
    return fmx_fail("fmx_dyt_step: bad sizes rows=%d cols=%d", rows, cols);
  if ((post_w == nullptr) != (post_b == nullptr) || (pre_w == nullptr) != (pre_b == nullptr))
    return fmx_fail("fmx_dyt_step: a dynamic tanh needs its weight and its bias");
  const long long n = (long long)rows * cols, cap = (long long)fmx_num_sms() * 16;
  const int block = 256;
  const int grid = (int)((n + block - 1) / block < cap ? (n + block - 1) / block : cap);
#define FMX_DYT(TY, TO)                                                                                              \
  fmx_launch(dyt_step_kernel<TY, TO>, dim3(grid), dim3(block), 0, stream, (const TY*)y, y_stride, post_alpha, post_w,  \
             post_b, mult, add, res_in, res_out, pre_alpha, pre_w, pre_b, (TO*)out, out_stride, (long long)rows, cols)
  const int yd = y != nullptr ? y_dtype : FMX_F32, od = out != nullptr ? out_dtype : FMX_F32;
  if (yd == FMX_F32 && od == FMX_F32) FMX_DYT(float, float);
  else if (yd == FMX_F32 && od == FMX_BF16) FMX_DYT(float, bf16);
  else if (yd == FMX_BF16 && od == FMX_F32) FMX_DYT(bf16, float);
  else if (yd == FMX_BF16 && od == FMX_BF16) FMX_DYT(bf16, bf16);
  else return fmx_fail("fmx_dyt_step: unknown dtypes %d, %d", y_dtype, out_dtype);
#undef FMX_DYT
  FMX_LAUNCH_CHECK();
  return 0;
}
