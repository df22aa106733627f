// Dynamic Tanh, a norm without statistics:  y = tanh(alpha * x) * w + b  with a scalar alpha
// and vectors w and b, optionally fused with the residual sum that precedes it and with the
// same transform of the summand:
//   d = delta[t,:]                                   (if delta)
//   d = tanh(alpha_d * d) * w_d + b_d                (if the summand has a norm of its own)
//   h[t,:] += d                                      (float32 sum, stored back unless rows gather)
//   out[t,:] = tanh(alpha * h[t,:]) * w + b          (if out)
// so that a layer of the form  h += norm_b(f(norm_a(h)))  costs one launch between two
// products.  All arithmetic is float32 (tanhf), the result is rounded once to the output type.
// alpha, w and b are float32 on the device (alpha a single float).  Elementwise: a token's
// result depends on nothing but its own row.
#include "common.cuh"

namespace {

struct DytParams {
  const float* alpha;  // one float
  const float* w;      // [dim]
  const float* b;      // [dim]
};

constexpr int DYT_THREADS = 256;

template <typename TD, typename TO>
__global__ void __launch_bounds__(DYT_THREADS)
dyt_kernel(float* h, const TD* delta, DytParams post, DytParams pre, TO* __restrict__ out,
           const int* __restrict__ rows, int dim) {
  // h and delta come from earlier kernels of the step: no __restrict__, loads stay below the wait
  pdl_trigger();
  const float a_pre = pre.alpha != nullptr ? pre.alpha[0] : 0.f;
  const float a_post = post.alpha != nullptr ? post.alpha[0] : 0.f;
  const int row = rows ? rows[blockIdx.x] : blockIdx.x;
  const bool store_h = delta != nullptr && rows == nullptr;
  pdl_wait();
  if (row < 0) return;
  const size_t base = (size_t)row * dim, obase = (size_t)blockIdx.x * dim;
  for (int d = threadIdx.x; d < dim; d += DYT_THREADS) {
    float v = h[base + d];
    if (delta != nullptr) {
      float e = to_f32<TD>(delta[base + d]);
      if (post.alpha != nullptr) e = fmaf(tanhf(a_post * e), post.w[d], post.b[d]);
      v += e;
      if (store_h) h[base + d] = v;
    }
    if (out != nullptr) out[obase + d] = from_f32<TO>(fmaf(tanhf(a_pre * v), pre.w[d], pre.b[d]));
  }
}

// Four elements a thread (16-byte accesses of the float32 stream) for dim % 4 == 0 and aligned
// rows; blockIdx.y walks a row's pieces.  Same arithmetic.
template <typename T>
__device__ __forceinline__ float4 dyt_load4(const T* p);
template <>
__device__ __forceinline__ float4 dyt_load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 dyt_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T>
__device__ __forceinline__ void dyt_store4(T* p, float4 v);
template <>
__device__ __forceinline__ void dyt_store4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void dyt_store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

__device__ __forceinline__ float4 dyt4(float4 v, float a, float4 w, float4 b) {
  return make_float4(fmaf(tanhf(a * v.x), w.x, b.x), fmaf(tanhf(a * v.y), w.y, b.y), fmaf(tanhf(a * v.z), w.z, b.z),
                     fmaf(tanhf(a * v.w), w.w, b.w));
}

template <typename TD, typename TO>
__global__ void __launch_bounds__(DYT_THREADS)
dyt_vec_kernel(float* h, const TD* delta, DytParams post, DytParams pre, TO* __restrict__ out,
               const int* __restrict__ rows, int dim) {
  pdl_trigger();
  const int d = (blockIdx.y * DYT_THREADS + threadIdx.x) * 4;
  const bool in_row = d < dim;
  // the norms' parameters and the row index do not depend on the kernels before this one
  const float a_pre = pre.alpha != nullptr ? pre.alpha[0] : 0.f;
  const float a_post = post.alpha != nullptr ? post.alpha[0] : 0.f;
  float4 w_pre = make_float4(0.f, 0.f, 0.f, 0.f), b_pre = w_pre, w_post = w_pre, b_post = w_pre;
  if (in_row && out != nullptr) {
    w_pre = *reinterpret_cast<const float4*>(pre.w + d);
    b_pre = *reinterpret_cast<const float4*>(pre.b + d);
  }
  if (in_row && post.alpha != nullptr) {
    w_post = *reinterpret_cast<const float4*>(post.w + d);
    b_post = *reinterpret_cast<const float4*>(post.b + d);
  }
  const int row = rows ? rows[blockIdx.x] : blockIdx.x;
  const bool store_h = delta != nullptr && rows == nullptr;
  pdl_wait();
  if (row < 0 || !in_row) return;
  const size_t base = (size_t)row * dim + d, obase = (size_t)blockIdx.x * dim + d;
  float4 v = *reinterpret_cast<const float4*>(h + base);
  if (delta != nullptr) {
    float4 e = dyt_load4<TD>(delta + base);
    if (post.alpha != nullptr) e = dyt4(e, a_post, w_post, b_post);
    v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w;
    if (store_h) *reinterpret_cast<float4*>(h + base) = v;
  }
  if (out != nullptr) dyt_store4<TO>(out + obase, dyt4(v, a_pre, w_pre, b_pre));
}

}  // namespace

// h: float32 [T, dim]; delta: [T, dim] of delta_dtype or null; post_*: the summand's own norm or
// null; pre_*: the norm of the sum (needed when out is given); out: [n_rows, dim] of out_dtype or
// null (null: only the sum is done); rows: null, or n_rows indices into h and delta to gather (h
// is then left as it was).
extern "C" int fg_dyt(void* h, const void* delta, int delta_dtype, const float* post_alpha, const float* post_w,
                      const float* post_b, const float* pre_alpha, const float* pre_w, const float* pre_b,
                      void* out, int out_dtype, const int* rows, int n_rows, int dim, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  FG_CHECK_ARG(dim > 0, "fg_dyt: bad dim %d", dim);
  FG_CHECK_ARG(out == nullptr || (pre_alpha && pre_w && pre_b), "fg_dyt: an output needs the norm's parameters");
  FG_CHECK_ARG(post_alpha == nullptr || (delta && post_w && post_b), "fg_dyt: the summand's norm needs a summand");
  FG_CHECK_ARG(out != nullptr || delta != nullptr, "fg_dyt: nothing to do");
  const DytParams post{post_alpha, post_w, post_b}, pre{pre_alpha, pre_w, pre_b};
  const auto aligned = [](const void* p) { return p == nullptr || ((uintptr_t)p & 15) == 0; };
  const bool vec = dim % 4 == 0 && aligned(h) && aligned(delta) && aligned(out) && aligned(post_w) && aligned(post_b) &&
                   aligned(pre_w) && aligned(pre_b) && (dim + 4 * DYT_THREADS - 1) / (4 * DYT_THREADS) <= 65535;
  const dim3 vec_grid(n_rows, (dim + 4 * DYT_THREADS - 1) / (4 * DYT_THREADS));
#define LAUNCH(TD, TO)                                                                                           \
  do {                                                                                                           \
    if (vec)                                                                                                     \
      fg_launch_pdl(dyt_vec_kernel<TD, TO>, vec_grid, dim3(DYT_THREADS), 0, stream, (float*)h, (const TD*)delta, \
                    post, pre, (TO*)out, rows, dim);                                                             \
    else                                                                                                         \
      fg_launch_pdl(dyt_kernel<TD, TO>, dim3(n_rows), dim3(DYT_THREADS), 0, stream, (float*)h, (const TD*)delta, \
                    post, pre, (TO*)out, rows, dim);                                                             \
  } while (0)
  const int key = (delta ? delta_dtype : FG_F32) * 2 + (out ? out_dtype : FG_F32);
  switch (key) {
    case 0: LAUNCH(float, float); break;
    case 1: LAUNCH(float, __nv_bfloat16); break;
    case 2: LAUNCH(__nv_bfloat16, float); break;
    case 3: LAUNCH(__nv_bfloat16, __nv_bfloat16); break;
    default: FG_CHECK_ARG(false, "fg_dyt: bad dtypes %d %d", delta_dtype, out_dtype);
  }
#undef LAUNCH
  FG_CHECK_LAUNCH("fg_dyt");
  return 0;
}
