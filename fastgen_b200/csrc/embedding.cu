// Token embedding: out[t, :] = table[token[t], :] * scale, written `copies` times side by
// side (out is [T, copies, dim]: a model with several residual streams starts them equal).
// Replaces F.embedding of fastgen/forward.py:403-410.  The output is the
// residual stream, which the engine keeps in float32 in every mode; the product with the
// scale is a float32 product.
#include "common.cuh"

template <typename TT, typename TO>
__global__ void embedding_kernel(const TT* __restrict__ table, const int* __restrict__ tokens,
                                 TO* __restrict__ out, int dim, int vocab, float scale, int copies,
                                 int* status) {
  const int t = blockIdx.x;
  int tok = tokens[t];
  TO* o = out + (size_t)t * copies * dim;
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0 && status) atomicOr(status, FG_STATUS_BAD_TOKEN);
    for (int d = threadIdx.x; d < copies * dim; d += blockDim.x) o[d] = from_f32<TO>(0.f);
    return;
  }
  const TT* row = table + (size_t)tok * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    const TO v = from_f32<TO>(to_f32<TT>(row[d]) * scale);
    for (int c = 0; c < copies; ++c) o[(size_t)c * dim + d] = v;
  }
}

extern "C" int fg_embedding(const void* table, int table_dtype, const int* tokens, void* out,
                            int out_dtype, int n_tokens, int dim, int vocab, float scale, int copies,
                            int* status, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(dim > 0 && vocab > 0 && copies > 0, "fg_embedding: bad sizes dim=%d vocab=%d copies=%d", dim, vocab,
               copies);
  const int threads = dim >= 1024 ? 256 : 128;
#define LAUNCH(TT, TO)                                                        \
  embedding_kernel<TT, TO><<<n_tokens, threads, 0, stream>>>(                 \
      (const TT*)table, tokens, (TO*)out, dim, vocab, scale, copies, status)
  if (table_dtype == FG_F32 && out_dtype == FG_F32) LAUNCH(float, float);
  else if (table_dtype == FG_BF16 && out_dtype == FG_F32) LAUNCH(__nv_bfloat16, float);
  else if (table_dtype == FG_BF16 && out_dtype == FG_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (table_dtype == FG_F32 && out_dtype == FG_BF16) LAUNCH(float, __nv_bfloat16);
  else FG_CHECK_ARG(false, "fg_embedding: bad dtypes %d %d", table_dtype, out_dtype);
#undef LAUNCH
  FG_CHECK_LAUNCH("fg_embedding");
  return 0;
}

// Token embedding plus a hashed bigram embedding:
//   out[t, :] = table[token[t], :] + bigram[row(t), :]
//   row(t) = (previous token * mul_prev + token * mul_cur) mod buckets, or `buckets` (the
//            table's last row) for a sequence's first token (position 0).
// The previous token of a token that opens its sequence's part of the step is the sequence's
// state: last_token[slot], which a second launch sets to the last token each sequence brings.
// Tokens of one sequence are consecutive in the step, so every other token finds its
// predecessor beside it.  Tokens of slot < 0 are padding: zeros, no state touched.
template <typename TT>
__global__ void embedding_bigram_kernel(const TT* __restrict__ table, const TT* __restrict__ bigram,
                                        const int* __restrict__ tokens, const int* __restrict__ pos,
                                        const int* __restrict__ req, const int* __restrict__ last_token,
                                        float* __restrict__ out, int dim, int vocab, int buckets, int mul_prev,
                                        int mul_cur, int* status) {
  const int t = blockIdx.x;
  const int slot = req[t];
  const int tok = tokens[t];
  float* o = out + (size_t)t * dim;
  if (slot < 0 || tok < 0 || tok >= vocab) {
    if (slot >= 0 && threadIdx.x == 0 && status) atomicOr(status, FG_STATUS_BAD_TOKEN);
    for (int d = threadIdx.x; d < dim; d += blockDim.x) o[d] = 0.f;
    return;
  }
  const int p = pos[t];
  long long row = buckets;
  if (p > 0) {
    const int prev = (t > 0 && req[t - 1] == slot) ? tokens[t - 1] : last_token[slot];
    row = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
    if (row < 0) row += buckets;
  }
  const TT* a = table + (size_t)tok * dim;
  const TT* b = bigram + (size_t)row * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) o[d] = to_f32<TT>(a[d]) + to_f32<TT>(b[d]);
}

__global__ void last_token_kernel(const int* __restrict__ tokens, const int* __restrict__ req,
                                  int* __restrict__ last_token, int n_tokens) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens) return;
  const int slot = req[t];
  if (slot < 0) return;
  if (t + 1 == n_tokens || req[t + 1] != slot) last_token[slot] = tokens[t];
}

extern "C" int fg_embedding_bigram(const void* table, const void* bigram, int table_dtype, const int* tokens,
                                   const int* pos, const int* req, int* last_token, float* out, int n_tokens,
                                   int dim, int vocab, int buckets, int mul_prev, int mul_cur, int* status,
                                   cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(dim > 0 && vocab > 0 && buckets > 0, "fg_embedding_bigram: bad sizes dim=%d vocab=%d buckets=%d", dim,
               vocab, buckets);
  const int threads = dim >= 1024 ? 256 : 128;
  if (table_dtype == FG_F32)
    embedding_bigram_kernel<float><<<n_tokens, threads, 0, stream>>>(
        (const float*)table, (const float*)bigram, tokens, pos, req, last_token, out, dim, vocab, buckets, mul_prev,
        mul_cur, status);
  else if (table_dtype == FG_BF16)
    embedding_bigram_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)table, (const __nv_bfloat16*)bigram, tokens, pos, req, last_token, out, dim, vocab,
        buckets, mul_prev, mul_cur, status);
  else
    FG_CHECK_ARG(false, "fg_embedding_bigram: bad dtype %d", table_dtype);
  FG_CHECK_LAUNCH("fg_embedding_bigram");
  last_token_kernel<<<(n_tokens + 255) / 256, 256, 0, stream>>>(tokens, req, last_token, n_tokens);
  FG_CHECK_LAUNCH("fg_embedding_bigram (state)");
  return 0;
}
