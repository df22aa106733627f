// Attention over a cached latent ("latent attention").
//
// A token caches one entry [c | k_t]: c, a latent of R numbers (RMS-normed), from which every
// head's keys and values are linear maps, and k_t, r numbers of one rotated key part that all
// heads share.  With the key map folded into the query (qa_h = U_k,h^T q_h, R numbers), head
// h's score for a key is (qa_h . c + qt_h . k_t) * scale, and its output is the softmax-weighted
// sum of the latents (R numbers), which the caller maps to values.  So the kernel is attention
// of H query heads on ONE key/value head whose keys are the entries and whose values are the
// entries' first R numbers.
//
// Here: the entry writer (norm, rotation, page write), the rotation of a part of every head,
// and the float32-arithmetic CUDA-core attention kernel, which serves prompt portions and single
// tokens alike.  Key tiles of 32 positions start at multiples of 32 from position 0, so the
// order of a row's sums depends on its own position only.
#include "common.cuh"

// ---- rotation of a part of each head ------------------------------------------------------------
// x[t, head, offset + 2i], x[t, head, offset + 2i + 1] turn by pos[t] * freqs[i]; cosine and sine
// are both multiplied by `magnitude`.  Angles are float32 products, sincosf is the precise one.
template <typename T>
__global__ void rotate_part_kernel(T* x, long stride, const int* __restrict__ pos, const int* __restrict__ req,
                                   const float* __restrict__ freqs, float magnitude, int n_heads, int head_size,
                                   int offset, int rot_dims) {
  const int t = blockIdx.x;
  if (req[t] < 0) return;
  const float p = (float)pos[t];
  const int pairs = rot_dims / 2;
  for (int i = threadIdx.x; i < n_heads * pairs; i += blockDim.x) {
    const int h = i / pairs, j = i - h * pairs;
    float sn, cs;
    sincosf(p * freqs[j], &sn, &cs);
    sn *= magnitude;
    cs *= magnitude;
    T* e = x + (size_t)t * stride + (size_t)h * head_size + offset + 2 * j;
    const float a = to_f32<T>(e[0]), b = to_f32<T>(e[1]);
    e[0] = from_f32<T>(a * cs - b * sn);
    e[1] = from_f32<T>(b * cs + a * sn);
  }
}

// ---- RMS norm of strided rows -----------------------------------------------------------------------
// out[t, :] = src[t, :] * rsqrt(mean(src[t, :]^2) + eps) * w for rows that are `stride` apart (the
// columns of one part of a wider product).
template <typename T>
__global__ void __launch_bounds__(128)
rms_rows_kernel(const T* __restrict__ src, long stride, const float* __restrict__ w, float eps, T* __restrict__ out,
                long out_stride, int dim) {
  __shared__ float scratch[32];
  const T* row = src + (size_t)blockIdx.x * stride;
  float ss = 0.f;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    const float v = to_f32<T>(row[d]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)dim + eps);
  for (int d = threadIdx.x; d < dim; d += blockDim.x)
    out[(size_t)blockIdx.x * out_stride + d] = from_f32<T>(to_f32<T>(row[d]) * rstd * w[d]);
}

extern "C" int fg_rms_rows(const void* src, long stride, int dtype, const float* w, float eps, void* out,
                           long out_stride, int n_rows, int dim, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  if (dtype == FG_F32)
    rms_rows_kernel<float><<<n_rows, 128, 0, stream>>>((const float*)src, stride, w, eps, (float*)out, out_stride, dim);
  else if (dtype == FG_BF16)
    rms_rows_kernel<__nv_bfloat16><<<n_rows, 128, 0, stream>>>((const __nv_bfloat16*)src, stride, w, eps,
                                                               (__nv_bfloat16*)out, out_stride, dim);
  else
    FG_CHECK_ARG(false, "fg_rms_rows: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_rms_rows");
  return 0;
}

// ---- the cache entry -----------------------------------------------------------------------------
// src[t] = [R latent numbers | r key numbers]; entry = [rmsnorm(latent) * w | rotated key part].
template <typename T>
__global__ void __launch_bounds__(128)
latent_entry_kernel(const T* __restrict__ src, long src_stride, const float* __restrict__ norm_w, float eps,
                    const float* __restrict__ freqs, float magnitude, T* __restrict__ pages,
                    const int* __restrict__ block_table, int table_width, int page_size, int n_pages,
                    const int* __restrict__ pos, const int* __restrict__ req, int R, int r, int E, int* status) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int slot = req[t];
  if (slot < 0) return;
  const int p = pos[t];
  const int logical = p / page_size;
  const int page = logical < table_width ? block_table[(size_t)slot * table_width + logical] : -1;
  if (page < 0 || page >= n_pages) {
    if (threadIdx.x == 0 && status) atomicOr(status, FG_STATUS_BAD_PAGE);
    return;
  }
  const T* row = src + (size_t)t * src_stride;
  T* entry = pages + ((size_t)page * page_size + (p - logical * page_size)) * E;
  float ss = 0.f;
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    const float v = to_f32<T>(row[d]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)R + eps);
  for (int d = threadIdx.x; d < R; d += blockDim.x) entry[d] = from_f32<T>(to_f32<T>(row[d]) * rstd * norm_w[d]);
  for (int j = threadIdx.x; j < r / 2; j += blockDim.x) {
    float sn, cs;
    sincosf((float)p * freqs[j], &sn, &cs);
    sn *= magnitude;
    cs *= magnitude;
    const float a = to_f32<T>(row[R + 2 * j]), b = to_f32<T>(row[R + 2 * j + 1]);
    entry[R + 2 * j] = from_f32<T>(a * cs - b * sn);
    entry[R + 2 * j + 1] = from_f32<T>(b * cs + a * sn);
  }
  for (int d = R + r + threadIdx.x; d < E; d += blockDim.x) entry[d] = from_f32<T>(0.f);
}

// ---- attention, CUDA cores, float32 arithmetic ------------------------------------------------------
constexpr int LA_ROWS = 16;   // (token, head) rows a block
constexpr int LA_KEYS = 32;   // key positions a tile
constexpr int LA_THREADS = 128;

template <typename T, typename TQ, int OD>
__global__ void __launch_bounds__(LA_THREADS)
latent_attention_simt_kernel(const TQ* __restrict__ qa, long qa_ts, long qa_hs, const T* __restrict__ qt, long qt_ts,
                             long qt_hs, T* __restrict__ out, long out_ts, long out_hs,
                             const T* __restrict__ gate, long gate_ts, const T* __restrict__ pages,
                             const int* __restrict__ block_table, int table_width, int page_size, int n_pages,
                             const int* __restrict__ pos, const int* __restrict__ tile_req,
                             const int* __restrict__ tile_tok0, const int* __restrict__ tile_ntok, int n_heads,
                             int heads_per_block, int R, int r, int E, float scale, int* status) {
  const int D = R + r, DP = D + 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* Qs = reinterpret_cast<float*>(smem_raw);  // [ROWS][DP]
  float* Ks = Qs + LA_ROWS * DP;                   // [KEYS][DP]
  float* Ps = Ks + LA_KEYS * DP;                   // [ROWS][KEYS + 1]
  __shared__ float alpha_s[LA_ROWS];
  __shared__ float l_s[LA_ROWS];
  __shared__ long long key_base[LA_KEYS];
  __shared__ int row_pos[LA_ROWS];

  const int tile = blockIdx.x, sub = blockIdx.y;
  const int b = tile_req[tile], tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto row_token = [&](int rr) { return rr / heads_per_block; };
  auto row_head = [&](int rr) { return sub * heads_per_block + (rr % heads_per_block); };
  auto row_valid = [&](int rr) { return row_token(rr) < ntok && row_head(rr) < n_heads; };
  const int o_row = tid >> 3, o_col = tid & 7;

  if (b < 0) {
    // padding of a fixed-size batch: no request, the output rows are zeroed
    if (row_valid(o_row)) {
      T* o = out + (size_t)(tok0 + row_token(o_row)) * out_ts + (size_t)row_head(o_row) * out_hs;
      for (int c = o_col; c < R; c += 8) o[c] = from_f32<T>(0.f);
    }
    return;
  }
  if (tid < LA_ROWS) row_pos[tid] = row_valid(tid) ? pos[tok0 + row_token(tid)] : -1;
  for (int i = tid; i < LA_ROWS * D; i += LA_THREADS) {
    const int rr = i / D, d = i - rr * D;
    float v = 0.f;
    if (row_valid(rr)) {
      const size_t tk = tok0 + row_token(rr), hh = row_head(rr);
      v = d < R ? to_f32<TQ>(qa[tk * qa_ts + hh * qa_hs + d]) : to_f32<T>(qt[tk * qt_ts + hh * qt_hs + (d - R)]);
    }
    Qs[rr * DP + d] = v;
  }
  __syncthreads();
  int max_pos = -1;
  for (int rr = 0; rr < LA_ROWS; ++rr) max_pos = max(max_pos, row_pos[rr]);
  if (max_pos < 0) return;

  float m_run[4], l_run[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m_run[i] = -INFINITY;
    l_run[i] = 0.f;
  }
  float o_acc[OD];
#pragma unroll
  for (int i = 0; i < OD; ++i) o_acc[i] = 0.f;

  for (int k0 = 0; k0 <= max_pos; k0 += LA_KEYS) {
    if (tid < LA_KEYS) {
      const int j = k0 + tid;
      long long base = -1;
      if (j <= max_pos) {
        const int logical = j / page_size;
        const int page = logical < table_width ? block_table[(size_t)b * table_width + logical] : -1;
        if (page >= 0 && page < n_pages)
          base = ((long long)page * page_size + (j - logical * page_size)) * E;
        else if (status)
          atomicOr(status, FG_STATUS_BAD_PAGE);
      }
      key_base[tid] = base;
    }
    __syncthreads();
    for (int i = tid; i < LA_KEYS * D; i += LA_THREADS) {
      const int c = i / D, d = i - c * D;
      const long long base = key_base[c];
      Ks[c * DP + d] = base >= 0 ? to_f32<T>(pages[base + d]) : 0.f;
    }
    __syncthreads();

    float s[4] = {0.f, 0.f, 0.f, 0.f};
    for (int d = 0; d < D; ++d) {
      const float kv = Ks[lane * DP + d];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] = fmaf(Qs[(warp + 4 * i) * DP + d], kv, s[i]);
    }
    const int j = k0 + lane;
    const bool has_key = key_base[lane] >= 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int rr = warp + 4 * i;
      const int p = row_pos[rr];
      const bool vis = has_key && p >= 0 && j <= p;
      const float sv = vis ? s[i] * scale : -INFINITY;
      const float m_new = fmaxf(m_run[i], warp_max(sv));
      float pr = 0.f, al = 1.f;
      if (m_new != -INFINITY) {
        pr = vis ? expf(sv - m_new) : 0.f;
        al = (m_run[i] == -INFINITY) ? 0.f : expf(m_run[i] - m_new);
      }
      l_run[i] = l_run[i] * al + warp_sum(pr);
      m_run[i] = m_new;
      Ps[rr * (LA_KEYS + 1) + lane] = pr;
      if (lane == 0) alpha_s[rr] = al;
    }
    __syncthreads();
    {
      const float al = alpha_s[o_row];
#pragma unroll
      for (int i = 0; i < OD; ++i) o_acc[i] *= al;
      for (int c = 0; c < LA_KEYS; ++c) {
        const float pr = Ps[o_row * (LA_KEYS + 1) + c];
#pragma unroll
        for (int i = 0; i < OD; ++i)
          if (o_col + 8 * i < R) o_acc[i] = fmaf(pr, Ks[c * DP + o_col + 8 * i], o_acc[i]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (lane == 0) l_s[warp + 4 * i] = l_run[i];
  __syncthreads();
  if (row_valid(o_row)) {
    const size_t tk = tok0 + row_token(o_row), hh = row_head(o_row);
    const float l = l_s[o_row];
    float f = l > 0.f ? 1.f / l : 0.f;
    if (gate != nullptr) f *= 1.f / (1.f + expf(-to_f32<T>(gate[tk * gate_ts + hh])));
    T* o = out + tk * out_ts + hh * out_hs;
#pragma unroll
    for (int i = 0; i < OD; ++i)
      if (o_col + 8 * i < R) o[o_col + 8 * i] = from_f32<T>(o_acc[i] * f);
  }
}

// ---- C interface -----------------------------------------------------------------------------------

extern "C" int fg_rotate_part(void* x, long stride, int dtype, const int* pos, const int* req, const float* freqs,
                              float magnitude, int n_tokens, int n_heads, int head_size, int offset, int rot_dims,
                              cudaStream_t stream) {
  if (n_tokens == 0 || rot_dims == 0) return 0;
  FG_CHECK_ARG(rot_dims % 2 == 0 && offset >= 0 && offset + rot_dims <= head_size,
               "fg_rotate_part: %d rotated dimensions at %d do not fit a head of %d", rot_dims, offset, head_size);
  if (dtype == FG_F32)
    rotate_part_kernel<float><<<n_tokens, 128, 0, stream>>>((float*)x, stride, pos, req, freqs, magnitude, n_heads,
                                                            head_size, offset, rot_dims);
  else if (dtype == FG_BF16)
    rotate_part_kernel<__nv_bfloat16><<<n_tokens, 128, 0, stream>>>((__nv_bfloat16*)x, stride, pos, req, freqs,
                                                                    magnitude, n_heads, head_size, offset, rot_dims);
  else
    FG_CHECK_ARG(false, "fg_rotate_part: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_rotate_part");
  return 0;
}

extern "C" int fg_latent_entry_write(const void* src, long src_stride, int dtype, const float* norm_w, float eps,
                                     const float* freqs, float magnitude, void* pages, const int* block_table,
                                     int table_width, int page_size, int n_pages, const int* pos, const int* req,
                                     int n_tokens, int R, int r, int E, int* status, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(R > 0 && r >= 0 && r % 2 == 0 && E >= R + r, "fg_latent_entry_write: bad sizes R=%d r=%d E=%d", R, r, E);
  if (dtype == FG_F32)
    latent_entry_kernel<float><<<n_tokens, 128, 0, stream>>>((const float*)src, src_stride, norm_w, eps, freqs,
                                                             magnitude, (float*)pages, block_table, table_width,
                                                             page_size, n_pages, pos, req, R, r, E, status);
  else if (dtype == FG_BF16)
    latent_entry_kernel<__nv_bfloat16><<<n_tokens, 128, 0, stream>>>(
        (const __nv_bfloat16*)src, src_stride, norm_w, eps, freqs, magnitude, (__nv_bfloat16*)pages, block_table,
        table_width, page_size, n_pages, pos, req, R, r, E, status);
  else
    FG_CHECK_ARG(false, "fg_latent_entry_write: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_latent_entry_write");
  return 0;
}

template <typename T, typename TQ>
static int launch_latent_simt(const void* qa, long qa_ts, long qa_hs, const void* qt, long qt_ts, long qt_hs, void* out,
                              long out_ts, long out_hs, const void* gate, long gate_ts, const void* pages,
                              const int* block_table, int table_width, int page_size, int n_pages, const int* pos,
                              const int* tile_req, const int* tile_tok0, const int* tile_ntok, int n_tiles,
                              int n_heads, int R, int r, int E, float scale, int* status, cudaStream_t stream) {
  const int hpb = n_heads < LA_ROWS ? n_heads : LA_ROWS;
  const dim3 grid(n_tiles, (n_heads + hpb - 1) / hpb);
  const int D = R + r;
  const size_t smem = sizeof(float) * ((size_t)(LA_ROWS + LA_KEYS) * (D + 1) + LA_ROWS * (LA_KEYS + 1));
  if (smem > 200 * 1024) {
    fg_set_error("fg_latent_attention_simt: entries of %d numbers do not fit shared memory", D);
    return -1;
  }
#define LA(OD)                                                                                                     \
  do {                                                                                                             \
    auto kern = latent_attention_simt_kernel<T, TQ, OD>;                                                           \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    kern<<<grid, LA_THREADS, smem, stream>>>((const TQ*)qa, qa_ts, qa_hs, (const T*)qt, qt_ts, qt_hs, (T*)out,     \
                                             out_ts, out_hs, (const T*)gate, gate_ts, (const T*)pages, block_table, \
                                             table_width, page_size, n_pages, pos, tile_req, tile_tok0, tile_ntok, \
                                             n_heads, hpb, R, r, E, scale, status);                                \
  } while (0)
  const int od = (R + 7) / 8;
  if (od <= 8) LA(8);
  else if (od <= 16) LA(16);
  else if (od <= 32) LA(32);
  else if (od <= 64) LA(64);
  else {
    fg_set_error("fg_latent_attention_simt: a latent of %d numbers is more than the kernel takes (512)", R);
    return -1;
  }
#undef LA
  return 0;
}

// Tiles hold LA_ROWS / min(heads, LA_ROWS) tokens each (the caller cuts them so).
extern "C" int fg_latent_attention_simt(const void* qa, int qa_dtype, long qa_ts, long qa_hs, const void* qt,
                                        long qt_ts, long qt_hs, void* out, long out_ts, long out_hs, int dtype,
                                        const void* gate, long gate_ts, const void* pages, const int* block_table,
                                        int table_width, int page_size, int n_pages, const int* pos,
                                        const int* tile_req, const int* tile_tok0, const int* tile_ntok, int n_tiles,
                                        int n_heads, int R, int r, int E, float scale, int* status,
                                        cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  FG_CHECK_ARG(n_heads > 0 && R > 0 && r >= 0 && E >= R + r, "fg_latent_attention_simt: bad sizes");
  int rc;
#define ARGS qa, qa_ts, qa_hs, qt, qt_ts, qt_hs, out, out_ts, out_hs, gate, gate_ts, pages, block_table, table_width, \
             page_size, n_pages, pos, tile_req, tile_tok0, tile_ntok, n_tiles, n_heads, R, r, E, scale, status, stream
  if (dtype == FG_F32 && qa_dtype == FG_F32) rc = launch_latent_simt<float, float>(ARGS);
  else if (dtype == FG_BF16 && qa_dtype == FG_F32) rc = launch_latent_simt<__nv_bfloat16, float>(ARGS);
  else if (dtype == FG_BF16 && qa_dtype == FG_BF16) rc = launch_latent_simt<__nv_bfloat16, __nv_bfloat16>(ARGS);
  else FG_CHECK_ARG(false, "fg_latent_attention_simt: bad dtypes %d %d", dtype, qa_dtype);
#undef ARGS
  if (rc) return rc;
  FG_CHECK_LAUNCH("fg_latent_attention_simt");
  return 0;
}
