// Paged attention with sigmoid weights on the CUDA cores, float32 arithmetic throughout.
//
//   out[i, h] = sum over visible j of  sigmoid(q_i . k_j * scale + gate[h] - r1[h] * ln(1 + r2[h] * (i - j))) * v_j
//
// The weight of a key is a sigmoid of its own score: nothing is normalised over the keys, so
// there is no running maximum, no rescaling and no division at the end.  gate is a number per
// query head added to the score; r1 and r2 (per head, both or neither) give a logarithmic
// distance bias that is taken off the score.  A key is visible if j <= i and, with a window,
// i - j < window.  Grouped-query heads h -> h / (Hq/Hkv).
//
// Tiling, paging and the order of the sums are those of attention_simt_kernel: a block takes
// one tile of query tokens for one group of heads, keys come from the cache pages in tiles of
// 32 positions that start at multiples of 32, and a key that is not visible adds an exact zero,
// so a row's result does not depend on how the prompt was cut or what else is in the batch.
//
// Storage type T (float or bf16) only affects loads and the final store.
//
// With tile_ntok == nullptr the list is one of single tokens (tile i is token tile_tok0[i] of
// request tile_req[i]); an entry without a request (negative) is then skipped, where a tile
// list's padding tile has its output rows zeroed.
#pragma once

#include "attention_simt.cuh"

namespace fg_attn {

template <typename T, int HD>
__global__ void __launch_bounds__(THREADS)
attention_sigmoid_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                         const int* __restrict__ block_table, int table_width, int page_size,
                         int n_pages, const int* __restrict__ pos, const int* __restrict__ tile_req,
                         const int* __restrict__ tile_tok0, const int* __restrict__ tile_ntok,
                         int n_kv_heads, int group, int heads_per_block, int window, float scale,
                         const float* __restrict__ gate, const float* __restrict__ r1,
                         const float* __restrict__ r2, int* status) {
  constexpr int HP = HD + 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float(*Qs)[HP] = reinterpret_cast<float(*)[HP]>(smem_raw);
  float(*Ks)[HP] = reinterpret_cast<float(*)[HP]>(Qs + ROWS);
  float(*Vs)[HP] = reinterpret_cast<float(*)[HP]>(Ks + KEYS);
  float(*Ps)[KEYS + 1] = reinterpret_cast<float(*)[KEYS + 1]>(Vs + KEYS);
  __shared__ long long key_base[KEYS];
  __shared__ int row_pos[ROWS];

  const int tile = blockIdx.x;
  const int g = blockIdx.y;        // key/value head
  const int sub = blockIdx.z;      // which slice of the group's heads
  const int b = tile_req[tile];
  const int tok0 = tile_tok0[tile];
  const int ntok = tile_ntok != nullptr ? tile_ntok[tile] : 1;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;

  auto row_token = [&](int r) { return r / heads_per_block; };
  auto row_head = [&](int r) { return sub * heads_per_block + (r % heads_per_block); };
  auto row_valid = [&](int r) { return row_token(r) < ntok && row_head(r) < group; };

  if (b < 0) {
    if (tile_ntok == nullptr) return;
    for (int i = tid; i < ROWS * HD; i += THREADS) {
      const int r = i / HD, d = i - r * HD;
      if (row_valid(r))
        out[(size_t)(tok0 + row_token(r)) * out_stride + (g * group + row_head(r)) * HD + d] = from_f32<T>(0.f);
    }
    return;
  }
  if (tid < ROWS) row_pos[tid] = row_valid(tid) ? pos[tok0 + row_token(tid)] : -1;
  for (int i = tid; i < ROWS * HD; i += THREADS) {
    const int r = i / HD, d = i - r * HD;
    float v = 0.f;
    if (row_valid(r))
      v = to_f32<T>(q[(size_t)(tok0 + row_token(r)) * q_stride + (g * group + row_head(r)) * HD + d]);
    Qs[r][d] = v;
  }
  __syncthreads();

  int max_pos = -1, min_pos = 0x7fffffff;
  for (int r = 0; r < ROWS; ++r) {
    const int p = row_pos[r];
    if (p >= 0) {
      max_pos = max(max_pos, p);
      min_pos = min(min_pos, p);
    }
  }
  if (max_pos < 0) return;
  int k_lo = 0;
  if (window > 0) k_lo = max(0, min_pos - window + 1) / KEYS * KEYS;

  // this thread's 4 score rows: warp, warp+4, warp+8, warp+12; column = lane.  Their heads' numbers:
  float g_row[4], r1_row[4], r2_row[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = warp + 4 * i;
    const int h = g * group + min(row_head(r), group - 1);
    g_row[i] = gate != nullptr ? gate[h] : 0.f;
    r1_row[i] = r1 != nullptr ? r1[h] : 0.f;
    r2_row[i] = r2 != nullptr ? r2[h] : 0.f;
  }
  constexpr int OD = HD / 8;
  float o_acc[OD];
#pragma unroll
  for (int i = 0; i < OD; ++i) o_acc[i] = 0.f;
  const int o_row = tid >> 3, o_col = tid & 7;

  for (int k0 = k_lo; k0 <= max_pos; k0 += KEYS) {
    if (tid < KEYS) {
      const int j = k0 + tid;
      long long base = -1;
      if (j <= max_pos) {
        const int logical = j / page_size;
        const int page = logical < table_width ? block_table[(size_t)b * table_width + logical] : -1;
        if (page >= 0 && page < n_pages) {
          base = (((long long)page * n_kv_heads + g) * page_size + (j - logical * page_size)) * HD;
        } else if (window <= 0 || j > min_pos - window) {
          if (status) atomicOr(status, FG_STATUS_BAD_PAGE);
        }
      }
      key_base[tid] = base;
    }
    __syncthreads();
    for (int i = tid; i < KEYS * HD; i += THREADS) {
      const int c = i / HD, d = i - c * HD;
      const long long base = key_base[c];
      float kv = 0.f, vv = 0.f;
      if (base >= 0) {
        kv = to_f32<T>(k_pages[base + d]);
        vv = to_f32<T>(v_pages[base + d]);
      }
      Ks[c][d] = kv;
      Vs[c][d] = vv;
    }
    __syncthreads();

    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
    for (int d = 0; d < HD; ++d) {
      const float kv = Ks[lane][d];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] = fmaf(Qs[warp + 4 * i][d], kv, s[i]);
    }
    const int j = k0 + lane;
    const bool has_key = key_base[lane] >= 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = warp + 4 * i;
      const int p = row_pos[r];
      const bool visible = has_key && p >= 0 && j <= p && (window <= 0 || j > p - window);
      float pr = 0.f;
      if (visible) {
        float z = s[i] * scale + g_row[i];
        if (r1 != nullptr) z -= r1_row[i] * logf(1.f + r2_row[i] * (float)(p - j));
        pr = 1.f / (1.f + expf(-z));
      }
      Ps[r][lane] = pr;
    }
    __syncthreads();
#pragma unroll 4
    for (int c = 0; c < KEYS; ++c) {
      const float pr = Ps[o_row][c];
#pragma unroll
      for (int i = 0; i < OD; ++i) o_acc[i] = fmaf(pr, Vs[c][o_col + 8 * i], o_acc[i]);
    }
    __syncthreads();
  }

  if (row_valid(o_row)) {
    T* o = out + (size_t)(tok0 + row_token(o_row)) * out_stride + (g * group + row_head(o_row)) * HD;
#pragma unroll
    for (int i = 0; i < OD; ++i) o[o_col + 8 * i] = from_f32<T>(o_acc[i]);
  }
}

// ---------------------------------------------------------------------------------
// Single tokens, bfloat16: the token's visible keys are cut into stretches of SIG_DECODE_KEYS
// positions that start at multiples of that number, and a block takes one stretch for one
// (token, key/value head): blockIdx.z counts the stretches from the first one the token sees,
// blocks beyond its last one leave at once.  A thread
// takes one key of the stretch: it reads the key's row and the value's row with 16-byte loads
// (all of a stretch's loads are in flight together: one round trip to memory a stretch), leaves
// the value in shared memory, forms the scores of the group's heads (float32, dimensions in
// ascending order) and leaves the weights in shared memory; then the threads turn to the
// output: thread (part, d) adds up weight * value over its part of the stretch's keys for
// dimension d, the parts are added in ascending order at the end.  Nothing is normalised, so
// a stretch's partial output is a plain sum: it goes to scratch [token, head, stretch, HD]
// (float32) and attention_sigmoid_combine_kernel adds a token's stretches in ascending order
// (with one stretch a launch, gridDim.z == 1, the block writes the output itself).  A token's
// result depends on its own position and window only.  Groups of more than SIG_DECODE_HEADS
// heads take passes.
// ---------------------------------------------------------------------------------
constexpr int SIG_DECODE_KEYS = 256;   // = threads
constexpr int SIG_DECODE_HEADS = 8;

template <int HD>
constexpr size_t sigmoid_decode_smem_bytes() {
  return sizeof(__nv_bfloat16) * SIG_DECODE_KEYS * HD;
}

template <int HD>
__global__ void __launch_bounds__(SIG_DECODE_KEYS)
attention_sigmoid_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                                int out_stride, const __nv_bfloat16* __restrict__ k_pages,
                                const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table,
                                int table_width, int page_size, int n_pages, const int* __restrict__ pos,
                                const int* __restrict__ seq_req, const int* __restrict__ seq_tok, int n_kv_heads,
                                int group, int window, float scale, const float* __restrict__ gate,
                                const float* __restrict__ r1, const float* __restrict__ r2, float* __restrict__ scratch,
                                int* status) {
  constexpr int PARTS = SIG_DECODE_KEYS / HD;                    // threads side by side on one dimension
  constexpr int PART_KEYS = (SIG_DECODE_KEYS + PARTS - 1) / PARTS;
  extern __shared__ __align__(16) unsigned char sig_smem[];
  __nv_bfloat16(*v_s)[HD] = reinterpret_cast<__nv_bfloat16(*)[HD]>(sig_smem);  // [SIG_DECODE_KEYS][HD]
  __shared__ float q_s[SIG_DECODE_HEADS][HD];
  __shared__ float w_s[SIG_DECODE_HEADS][SIG_DECODE_KEYS];
  __shared__ float part_s[PARTS][SIG_DECODE_HEADS][HD];
  const int b = seq_req[blockIdx.x];
  if (b < 0) return;
  const int tok = seq_tok[blockIdx.x];
  const int g = blockIdx.y;
  const int tid = threadIdx.x;
  const int p = pos[tok];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int part = tid / HD, d = tid - part * HD;
  const int k0 = (lo / SIG_DECODE_KEYS + (int)blockIdx.z) * SIG_DECODE_KEYS;
  if (k0 > p) return;
  if (gridDim.z == 1 && k0 + SIG_DECODE_KEYS <= p) {
    // the launch was sized for fewer stretches than this token has
    if (tid == 0 && status) atomicOr(status, FG_STATUS_BAD_SPLITS);
    return;
  }
  for (int h0 = 0; h0 < group; h0 += SIG_DECODE_HEADS) {
    const int nh = min(SIG_DECODE_HEADS, group - h0);
    for (int i = tid; i < nh * HD; i += SIG_DECODE_KEYS) {
      const int h = i / HD, dd = i - h * HD;
      q_s[h][dd] = __bfloat162float(q[(size_t)tok * q_stride + (g * group + h0 + h) * HD + dd]);
    }
    float acc[SIG_DECODE_HEADS];
#pragma unroll
    for (int h = 0; h < SIG_DECODE_HEADS; ++h) acc[h] = 0.f;
    __syncthreads();
    {
      const int j = k0 + tid;
      long long base = -1;
      if (j >= lo && j <= p) {
        const int logical = j / page_size;
        const int page = logical < table_width ? block_table[(size_t)b * table_width + logical] : -1;
        if (page >= 0 && page < n_pages)
          base = (((long long)page * n_kv_heads + g) * page_size + (j - logical * page_size)) * HD;
        else if (status)
          atomicOr(status, FG_STATUS_BAD_PAGE);
      }
      float s[SIG_DECODE_HEADS];
#pragma unroll
      for (int h = 0; h < SIG_DECODE_HEADS; ++h) s[h] = 0.f;
      uint4* v_row = reinterpret_cast<uint4*>(&v_s[tid][0]);
      if (base >= 0) {
        const uint4* k_row = reinterpret_cast<const uint4*>(k_pages + base);
        const uint4* v_src = reinterpret_cast<const uint4*>(v_pages + base);
#pragma unroll
        for (int c = 0; c < HD / 8; ++c) v_row[c] = v_src[c];
#pragma unroll
        for (int c = 0; c < HD / 8; ++c) {
          const uint4 raw = k_row[c];
          const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 kv = __bfloat1622float2(k2[e]);
#pragma unroll
            for (int h = 0; h < SIG_DECODE_HEADS; ++h) {
              if (h < nh) {
                s[h] = fmaf(q_s[h][c * 8 + 2 * e], kv.x, s[h]);
                s[h] = fmaf(q_s[h][c * 8 + 2 * e + 1], kv.y, s[h]);
              }
            }
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < HD / 8; ++c) v_row[c] = make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int h = 0; h < SIG_DECODE_HEADS; ++h) {
        if (h < nh) {
          float wgt = 0.f;
          if (base >= 0) {
            const int head = g * group + h0 + h;
            float z = s[h] * scale + (gate != nullptr ? gate[head] : 0.f);
            if (r1 != nullptr) z -= r1[head] * logf(1.f + r2[head] * (float)(p - j));
            wgt = 1.f / (1.f + expf(-z));
          }
          w_s[h][tid] = wgt;
        }
      }
      __syncthreads();
      if (part < PARTS) {
        const int j_end = min(SIG_DECODE_KEYS, (part + 1) * PART_KEYS);
#pragma unroll 4
        for (int jj = part * PART_KEYS; jj < j_end; ++jj) {
          const float vv = __bfloat162float(v_s[jj][d]);
#pragma unroll
          for (int h = 0; h < SIG_DECODE_HEADS; ++h)
            if (h < nh) acc[h] = fmaf(w_s[h][jj], vv, acc[h]);
        }
      }
      __syncthreads();
    }
    if (part < PARTS) {
#pragma unroll
      for (int h = 0; h < SIG_DECODE_HEADS; ++h)
        if (h < nh) part_s[part][h][d] = acc[h];
    }
    __syncthreads();
    for (int i = tid; i < nh * HD; i += SIG_DECODE_KEYS) {
      const int h = i / HD, dd = i - h * HD;
      float total = 0.f;
#pragma unroll
      for (int pt = 0; pt < PARTS; ++pt) total += part_s[pt][h][dd];
      const int head = g * group + h0 + h;
      if (gridDim.z == 1)
        out[(size_t)tok * out_stride + head * HD + dd] = __float2bfloat16_rn(total);
      else
        scratch[(((size_t)blockIdx.x * (n_kv_heads * group) + head) * gridDim.z + blockIdx.z) * HD + dd] = total;
    }
    __syncthreads();
  }
}

// out[token, head, :] = the sum of the token's stretches, in ascending order.  One block per
// (token, head); the number of stretches follows from the token's position and the window.
template <int HD>
__global__ void attention_sigmoid_combine_kernel(__nv_bfloat16* __restrict__ out, int out_stride,
                                                 const int* __restrict__ pos, const int* __restrict__ seq_req,
                                                 const int* __restrict__ seq_tok, int n_heads, int window,
                                                 int max_stretches, const float* scratch, int* status) {
  if (seq_req[blockIdx.x] < 0) return;
  const int tok = seq_tok[blockIdx.x];
  const int head = blockIdx.y;
  const int p = pos[tok];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  int n = p / SIG_DECODE_KEYS - lo / SIG_DECODE_KEYS + 1;
  if (n > max_stretches) {
    if (threadIdx.x == 0 && status) atomicOr(status, FG_STATUS_BAD_SPLITS);
    n = max_stretches;
  }
  const float* src = scratch + ((size_t)blockIdx.x * n_heads + head) * max_stretches * HD;
  for (int dd = threadIdx.x; dd < HD; dd += blockDim.x) {
    float total = 0.f;
    for (int z = 0; z < n; ++z) total += src[(size_t)z * HD + dd];
    out[(size_t)tok * out_stride + head * HD + dd] = __float2bfloat16_rn(total);
  }
}

}  // namespace fg_attn
