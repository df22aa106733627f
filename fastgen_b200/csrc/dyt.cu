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
#define LAUNCH(TD, TO)                                                                                  \
  fg_launch_pdl(dyt_kernel<TD, TO>, dim3(n_rows), dim3(DYT_THREADS), 0, stream, (float*)h, (const TD*)delta, \
                post, pre, (TO*)out, rows, dim)
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
