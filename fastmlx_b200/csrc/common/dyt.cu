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
// The same, four neighbouring columns per thread in 16-byte (bfloat16: 8-byte) accesses.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<unsigned*>(&a);
  u.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ float4 dyt4(float4 v, float alpha, float4 w, float4 b) {
  return make_float4(fmaf(tanhf(alpha * v.x), w.x, b.x), fmaf(tanhf(alpha * v.y), w.y, b.y), fmaf(tanhf(alpha * v.z), w.z, b.z),
                     fmaf(tanhf(alpha * v.w), w.w, b.w));
}

template <typename TY, typename TO>
__global__ void dyt_step_vec_kernel(const TY* y, long long y_stride, float post_alpha, const float* __restrict__ post_w,
                                    const float* __restrict__ post_b, float mult, const float* __restrict__ add,
                                    const float* res_in, float* res_out, float pre_alpha, const float* __restrict__ pre_w,
                                    const float* __restrict__ pre_b, TO* out, long long out_stride, long long rows, int cols) {
  pdl_wait();
  pdl_trigger();
  const int c4 = cols / 4;
  const long long n = rows * c4;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / c4;
    const int c = (int)(idx - r * c4) * 4;
    float4 s = res_in != nullptr ? load4(res_in + r * cols + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (y != nullptr) {
      float4 v = load4(y + r * y_stride + c);
      if (post_w != nullptr) v = dyt4(v, post_alpha, load4(post_w + c), load4(post_b + c));
      s = make_float4(fmaf(mult, v.x, s.x), fmaf(mult, v.y, s.y), fmaf(mult, v.z, s.z), fmaf(mult, v.w, s.w));
    }
    if (add != nullptr) {
      const float4 a = load4(add + c);
      s = make_float4(s.x + a.x, s.y + a.y, s.z + a.z, s.w + a.w);
    }
    if (res_out != nullptr) store4(res_out + r * cols + c, s);
    if (out != nullptr) store4(out + r * out_stride + c, pre_w != nullptr ? dyt4(s, pre_alpha, load4(pre_w + c), load4(pre_b + c)) : s);
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
  // four columns per thread where every row and vector starts on 16 bytes (the arithmetic is the same element by element)
  auto a16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = cols % 4 == 0 && y_stride % 8 == 0 && out_stride % 8 == 0 && a16(y) && a16(out) && a16(res_in) && a16(res_out) &&
                   a16(post_w) && a16(post_b) && a16(pre_w) && a16(pre_b) && a16(add);
  const long long n = (long long)rows * (vec ? cols / 4 : cols), cap = (long long)fmx_num_sms() * 16;
  const int block = 256;
  const int grid = (int)((n + block - 1) / block < cap ? (n + block - 1) / block : cap);
#define FMX_DYT(TY, TO)                                                                                              \
  do {                                                                                                               \
    if (vec)                                                                                                         \
      fmx_launch(dyt_step_vec_kernel<TY, TO>, dim3(grid), dim3(block), 0, stream, (const TY*)y, y_stride, post_alpha, post_w, \
                 post_b, mult, add, res_in, res_out, pre_alpha, pre_w, pre_b, (TO*)out, out_stride, (long long)rows, cols); \
    else                                                                                                             \
      fmx_launch(dyt_step_kernel<TY, TO>, dim3(grid), dim3(block), 0, stream, (const TY*)y, y_stride, post_alpha, post_w, \
                 post_b, mult, add, res_in, res_out, pre_alpha, pre_w, pre_b, (TO*)out, out_stride, (long long)rows, cols); \
  } while (0)
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
