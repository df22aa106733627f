// Norms with mean and variance (layer norm) or without (RMS), over one residual stream or
// over several that are mixed on the way ("hyper-connections"), fused with the sum that
// precedes them.  For a row (token) with streams x_0 .. x_{S-1} (float32, stored [T, S, dim]):
//
//   if delta:  x_t <- sum_s mix[s, t] * x_s + out_coef[t] * delta      (all t from the old x_s)
//   u = sum_s in_coef[s] * x_s
//   out = (u - mean(u)) * rsqrt(var(u) + eps) * w + b                  (kind 0: layer norm)
//   out = u * rsqrt(mean(u^2) + eps) * w                               (kind 1: RMS norm)
//
// Null coefficient pointers stand for the identity mix and for coefficients of one, so S = 1
// with null pointers is the ordinary "h += delta; out = norm(h)".  All arithmetic is float32;
// the variance is the mean of the squared deviations from the mean (two passes over the row,
// which waits in shared memory).  One block a row; the order of every sum depends on dim and
// the block size only.  With `rows`, output row i comes from input row rows[i] and the
// streams are not stored back.
#include "common.cuh"

constexpr int SN_MAX_STREAMS = 8;
constexpr int SN_THREADS = 256;

// S is the number of streams when it is 1 to 4 (the loops over streams unroll to what is needed),
// 0 for any number up to SN_MAX_STREAMS.
template <typename TD, typename TO, int S_>
__global__ void __launch_bounds__(SN_THREADS)
stream_norm_kernel(float* h, int n_streams, const TD* delta, const float* __restrict__ mix,
                   const float* __restrict__ out_coef, const float* __restrict__ in_coef,
                   const float* __restrict__ w, const float* __restrict__ b, TO* __restrict__ out,
                   const int* rows, int dim, float eps, int kind) {
  extern __shared__ float u_s[];
  __shared__ float scratch[32];
  constexpr int SM = S_ > 0 ? S_ : SN_MAX_STREAMS;  // bound of the unrolled loops
  const int S = S_ > 0 ? S_ : n_streams;
  pdl_trigger();
  // the coefficients are the model's: read (into registers, the loops below are unrolled) while
  // the kernel before this one finishes; the streams and the summand are touched after the wait
  float mx[SM][SM], oc[SM], ic[SM];
#pragma unroll
  for (int a = 0; a < SM; ++a) {
    oc[a] = (a < S && out_coef) ? out_coef[a] : (a < S ? 1.f : 0.f);
    ic[a] = (a < S && in_coef) ? in_coef[a] : (a < S ? 1.f : 0.f);
#pragma unroll
    for (int c = 0; c < SM; ++c) mx[a][c] = (a < S && c < S) ? (mix ? mix[a * S + c] : (a == c ? 1.f : 0.f)) : 0.f;
  }
  // a row of up to 8 x 256 columns: its weights wait in registers too
  const bool small = dim <= 8 * SN_THREADS;
  float w_r[8], b_r[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int d = threadIdx.x + i * SN_THREADS;
    w_r[i] = (small && out != nullptr && d < dim) ? w[d] : 0.f;
    b_r[i] = (small && out != nullptr && b != nullptr && d < dim) ? b[d] : 0.f;
  }
  const int* rows_v = rows;
  pdl_wait();
  const size_t row = rows_v ? ld_global_4(rows_v + blockIdx.x) : blockIdx.x;
  float* x = h + row * (size_t)S * dim;
  const bool store = delta != nullptr && rows == nullptr;
  const bool has_mix = mix != nullptr, has_in = in_coef != nullptr;
  float sum = 0.f;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float xs[SM];
#pragma unroll
    for (int s = 0; s < SM; ++s) xs[s] = s < S ? x[(size_t)s * dim + d] : 0.f;
    float u = 0.f;
    if (delta != nullptr) {
      const float y = to_f32<TD>(delta[row * dim + d]);
#pragma unroll
      for (int t = 0; t < SM; ++t) {
        if (t < S) {
          float v = 0.f;
          if (!has_mix) {
            v = xs[t];
          } else {
#pragma unroll
            for (int s = 0; s < SM; ++s)
              if (s < S) v = fmaf(mx[s][t], xs[s], v);
          }
          v = fmaf(oc[t], y, v);
          if (store) x[(size_t)t * dim + d] = v;
          u = has_in ? fmaf(ic[t], v, u) : u + v;
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < SM; ++t)
        if (t < S) u = has_in ? fmaf(ic[t], xs[t], u) : u + xs[t];
    }
    u_s[d] = u;
    sum += kind == 0 ? u : u * u;
  }
  if (out == nullptr) return;
  sum = block_sum(sum, scratch);
  float mean = 0.f, rstd;
  if (kind == 0) {
    mean = sum / (float)dim;
    float sq = 0.f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      const float c = u_s[d] - mean;
      sq += c * c;
    }
    sq = block_sum(sq, scratch);
    rstd = 1.f / sqrtf(sq / (float)dim + eps);
  } else {
    rstd = 1.f / sqrtf(sum / (float)dim + eps);
  }
  TO* o = out + (size_t)blockIdx.x * dim;
  if (small) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = threadIdx.x + i * SN_THREADS;
      if (d < dim) o[d] = from_f32<TO>((u_s[d] - mean) * rstd * w_r[i] + b_r[i]);
    }
    return;
  }
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float v = (u_s[d] - mean) * rstd * w[d];
    if (b != nullptr) v += b[d];
    o[d] = from_f32<TO>(v);
  }
}

extern "C" int fg_stream_norm(float* h, int n_streams, const void* delta, int delta_dtype, const float* mix,
                              const float* out_coef, const float* in_coef, const float* w, const float* b,
                              void* out, int out_dtype, const int* rows, int n_rows, int dim, float eps, int kind,
                              cudaStream_t stream) {
  if (n_rows == 0) return 0;
  FG_CHECK_ARG(n_streams >= 1 && n_streams <= SN_MAX_STREAMS, "fg_stream_norm: %d streams (at most %d)", n_streams,
               SN_MAX_STREAMS);
  FG_CHECK_ARG(dim > 0 && (kind == 0 || kind == 1), "fg_stream_norm: bad dim %d or kind %d", dim, kind);
  FG_CHECK_ARG(out == nullptr || w != nullptr, "fg_stream_norm: a norm needs its weight");
  const size_t smem = sizeof(float) * (size_t)dim;
  FG_CHECK_ARG(smem <= 200 * 1024, "fg_stream_norm: a row of %d does not fit shared memory", dim);
#define LAUNCH_S(TD, TO, S)                                                                                  \
  do {                                                                                                       \
    auto kern = stream_norm_kernel<TD, TO, S>;                                                               \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    fg_launch_pdl(kern, dim3(n_rows), dim3(SN_THREADS), smem, stream, h, n_streams, (const TD*)delta, mix,   \
                  out_coef, in_coef, w, b, (TO*)out, rows, dim, eps, kind);                                  \
  } while (0)
#define LAUNCH(TD, TO)                          \
  do {                                          \
    if (n_streams == 1) LAUNCH_S(TD, TO, 1);    \
    else if (n_streams == 2) LAUNCH_S(TD, TO, 2); \
    else if (n_streams == 3) LAUNCH_S(TD, TO, 3); \
    else if (n_streams == 4) LAUNCH_S(TD, TO, 4); \
    else LAUNCH_S(TD, TO, 0);                   \
  } while (0)
  const bool df = delta == nullptr || delta_dtype == FG_F32;
  if (df && out_dtype == FG_F32) LAUNCH(float, float);
  else if (df && out_dtype == FG_BF16) LAUNCH(float, __nv_bfloat16);
  else if (!df && out_dtype == FG_F32) LAUNCH(__nv_bfloat16, float);
  else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
#undef LAUNCH_S
  FG_CHECK_LAUNCH("fg_stream_norm");
  return 0;
}
