// Attention over a cached latent on the tensor cores (bfloat16, mma.sync m16n8k16), compiled
// per latent size: -DFG_LATENT_RANK=R -DFG_LATENT_ROT=r.
//
// The computation of latent.cu: H query heads attend to ONE entry [c (R) | k_t (r)] per cached
// token; the score is (qa_h . c + qt_h . k_t) * scale, the output the softmax-weighted sum of
// the c, times sigmoid(gate) when a gate is given.  A key tile in shared memory is therefore
// both the K operand (all D = R + r columns) and the V operand (its first R columns): it is
// loaded once.
//
// A block takes 64 (token, head) rows of one attention tile and, when the launch is split,
// one stretch of its keys.  Four row warps own 16 rows each; with latents above 256 numbers a
// second set of four warps owns the other half of the output columns (both sets compute the
// scores).  Keys come in tiles of 64 (32 for entries above 400 numbers) through a two-stage
// cp.async ring.  Softmax statistics and the output accumulators are float32; the
// probabilities are rounded to bfloat16 for the second product.
//
// Few tiles (single tokens above all) leave most of the GPU idle, so the host may cut every
// tile's keys into `n_splits` stretches of `keys_per_split` positions: each (tile, stretch)
// block leaves an unnormalised partial with its maximum and sum, and a second kernel merges
// the stretches in ascending order, applies the gate and stores.  The stretches are fixed
// multiples of the key tile from position 0, so a row's result does not depend on the batch.
#include "attention_mma.cuh"

#ifndef FG_LATENT_RANK
#error "compile with -DFG_LATENT_RANK and -DFG_LATENT_ROT"
#endif

namespace fg_latent {
using namespace fg_mma;

constexpr int R = FG_LATENT_RANK, ROT = FG_LATENT_ROT;
constexpr int D = R + ROT;
constexpr int E = (D + 7) / 8 * 8;       // numbers of a cache entry (16-byte multiple)
constexpr int D16 = (D + 15) / 16 * 16;  // columns of the shared-memory tiles
constexpr int R16 = (R + 15) / 16 * 16;
constexpr int WN = R16 <= 256 ? 1 : 2;   // sets of warps over the output columns
constexpr int RW = R16 / WN;             // output columns a warp owns
constexpr int LD = D16 + 8;
constexpr int ROWS = 64;
constexpr int KEYS = D16 <= 400 ? 64 : 32;
constexpr int NT = KEYS / 8;
constexpr int NTHREADS = 128 * WN;
constexpr int PART = R16 + 2;            // floats of a partial: the output, then maximum and sum
constexpr int MERGE_SPLITS = 256;        // most stretches a launch may be cut into
static_assert(R % 8 == 0 && ROT % 2 == 0, "latents are multiples of 8, rotated parts of 2");
static_assert(RW % 16 == 0, "a warp's output columns come in sixteens");

constexpr size_t smem_bytes() { return sizeof(__nv_bfloat16) * (size_t)LD * (ROWS + 2 * KEYS); }

__global__ void __launch_bounds__(NTHREADS)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ qa, long qa_ts, long qa_hs,
                            const __nv_bfloat16* __restrict__ qt, long qt_ts, long qt_hs,
                            __nv_bfloat16* __restrict__ out, long out_ts, long out_hs,
                            const __nv_bfloat16* __restrict__ gate, long gate_ts,
                            const __nv_bfloat16* __restrict__ pages, const int* __restrict__ block_table,
                            int table_width, int page_size, int n_pages, const int* __restrict__ pos,
                            const int* __restrict__ tile_req, const int* __restrict__ tile_tok0,
                            const int* __restrict__ tile_ntok, int n_heads, int heads_per_block, float scale_log2,
                            int n_splits, int keys_per_split, float* __restrict__ scratch, int* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Ks = Qs + ROWS * LD;  // 2 stages
  __shared__ int row_pos[ROWS];
  __shared__ long long row_off[2][KEYS];

  const int tile = blockIdx.x, sub = blockIdx.y, split = blockIdx.z;
  const int b = tile_req[tile];
  const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int warp_m = warp & 3, warp_n = warp >> 2;
  auto row_token = [&](int r) { return r / heads_per_block; };
  auto row_head = [&](int r) { return sub * heads_per_block + (r % heads_per_block); };
  auto row_valid = [&](int r) { return row_token(r) < ntok && row_head(r) < n_heads; };
  float* part_base = scratch + ((size_t)(tile * gridDim.y + sub) * ROWS) * n_splits * PART;

  if (b < 0) {
    // a tile of no request (padding of a captured step): its rows, if it names any, are zeroed
    if (n_splits == 1)
      for (int i = tid; i < ROWS * (R / 2); i += NTHREADS) {
        const int r = i / (R / 2), c = i - r * (R / 2);
        if (row_valid(r))
          *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(tok0 + row_token(r)) * out_ts +
                                             (size_t)row_head(r) * out_hs + 2 * c) = __floats2bfloat162_rn(0.f, 0.f);
      }
    return;
  }
  if (tid < ROWS) row_pos[tid] = row_valid(tid) ? pos[tok0 + row_token(tid)] : -1;
  // queries -> shared memory: [qa | qt | zeros], zero rows where the tile is not full; asynchronous
  // 4-byte copies, all in flight at once (a tile of single tokens is mostly this load)
  for (int i = tid; i < ROWS * (D16 / 2); i += NTHREADS) {
    const int r = i / (D16 / 2), col = 2 * (i - r * (D16 / 2));
    const bool ok = row_valid(r) && col < D;
    const __nv_bfloat16* src = qa;
    if (ok) {
      const size_t tk = tok0 + row_token(r), hh = row_head(r);
      src = col < R ? qa + tk * qa_ts + hh * qa_hs + col : qt + tk * qt_ts + hh * qt_hs + (col - R);
    }
    const int bytes = ok ? 4 : 0;  // 0: zero-filled, nothing is read
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(smem_u32(Qs + r * LD + col)), "l"(src), "r"(bytes)
                 : "memory");
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  int max_pos = -1;
  for (int r = 0; r < ROWS; r += heads_per_block) max_pos = max(max_pos, row_pos[r]);  // rows are ordered by token
  const int k_first = split * keys_per_split;
  const int k_end = min(max_pos + 1, k_first + keys_per_split);
  const int n_tiles = k_end > k_first ? (k_end - k_first + KEYS - 1) / KEYS : 0;
  const int* table_row = block_table + (size_t)b * table_width;

  auto offsets = [&](int t) {
    kv_row_offsets<E>(row_off[t & 1], table_row, table_width, page_size, n_pages, 1, 0, k_first + t * KEYS, KEYS,
                      k_first, k_end, tid, status);
  };
  auto issue = [&](int t) {
    const int stage = t & 1;
    __nv_bfloat16* dst = Ks + stage * KEYS * LD;
    constexpr int CH = D16 / 8;
    for (int i = tid; i < KEYS * CH; i += NTHREADS) {
      const int r = i / CH, c = i - r * CH;
      const long long off = row_off[stage][r];
      const bool ok = off >= 0 && c * 8 < E;
      cp_async_16(dst + r * LD + c * 8, ok ? pages + off + c * 8 : pages, ok);
    }
    cp_async_commit();
  };
  if (n_tiles > 0) {
    offsets(0);
    __syncthreads();
    issue(0);
    if (n_tiles > 1) offsets(1);
  }
  __syncthreads();  // tile 1's offsets are read by every thread when its copies are issued

  const int r0 = warp_m * 16 + (lane >> 2), r1 = r0 + 8;
  const int p0 = row_pos[r0], p1 = row_pos[r1];
  int warp_max = -1;
  for (int r = warp_m * 16; r < warp_m * 16 + 16; ++r) warp_max = max(warp_max, row_pos[r]);

  float o[RW / 8][4];
#pragma unroll
  for (int i = 0; i < RW / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int t = 0; t < n_tiles; ++t) {
    if (t + 1 < n_tiles) {
      issue(t + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (t + 2 < n_tiles) offsets(t + 2);
    const int k0 = k_first + t * KEYS;
    if (k0 <= warp_max) {
      const __nv_bfloat16* ks = Ks + (t & 1) * KEYS * LD;
      float s[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll 4
      for (int kk = 0; kk < D16 / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, Qs + (warp_m * 16 + (lane & 15)) * LD + kk * 16 + ((lane >> 4) << 3));
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          uint32_t bq[4];
          const int key = np * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int dim = kk * 16 + (((lane >> 3) & 1) << 3);
          ldmatrix_x4(bq, ks + key * LD + dim);
          mma_16816(s[2 * np], a, bq[0], bq[1]);
          mma_16816(s[2 * np + 1], a, bq[2], bq[3]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = k0 + nt * 8 + 2 * (lane & 3) + (e & 1);
          const int p = (e < 2) ? p0 : p1;
          const bool vis = p >= 0 && j <= p && j < k_end;
          s[nt][e] = vis ? s[nt][e] * scale_log2 : -INFINITY;
        }
      softmax_step<RW, NT>(s, o, m, l);
      // the tile's first R columns are the values; this warp's share starts at warp_n * RW
#pragma unroll
      for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int np = 0; np < RW / 16; ++np) {
          uint32_t bv[4];
          const int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int dim = warp_n * RW + np * 16 + ((lane >> 4) << 3);
          ldmatrix_x4_trans(bv, ks + key * LD + dim);
          mma_16816(o[2 * np], a, bv[0], bv[1]);
          mma_16816(o[2 * np + 1], a, bv[2], bv[3]);
        }
      }
    }
    __syncthreads();  // everyone is done with this stage before it is refilled
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = h ? r1 : r0;
    if (!row_valid(r)) continue;
    const size_t tk = tok0 + row_token(r), hh = row_head(r);
    if (n_splits > 1) {
      float* dst = part_base + ((size_t)r * n_splits + split) * PART;
#pragma unroll
      for (int nt = 0; nt < RW / 8; ++nt) {
        const int d = warp_n * RW + nt * 8 + 2 * (lane & 3);
        *reinterpret_cast<float2*>(dst + d) = make_float2(o[nt][2 * h], o[nt][2 * h + 1]);
      }
      if (warp_n == 0 && (lane & 3) == 0) {
        dst[R16] = m[h];
        dst[R16 + 1] = l[h];
      }
      continue;
    }
    float f = l[h] > 0.f ? 1.f / l[h] : 0.f;
    if (gate != nullptr) f *= 1.f / (1.f + __expf(-__bfloat162float(gate[tk * gate_ts + hh])));
    __nv_bfloat16* dst = out + tk * out_ts + hh * out_hs;
#pragma unroll
    for (int nt = 0; nt < RW / 8; ++nt) {
      const int d = warp_n * RW + nt * 8 + 2 * (lane & 3);
      if (d < R) *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(o[nt][2 * h] * f, o[nt][2 * h + 1] * f);
    }
  }
}

// The stretches of a row, merged in ascending order: out = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m),
// times the gate.  One block a (tile, head slice, row).
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ scratch, __nv_bfloat16* __restrict__ out, long out_ts, long out_hs,
                    const __nv_bfloat16* __restrict__ gate, long gate_ts, const int* __restrict__ tile_req,
                    const int* __restrict__ tile_tok0, const int* __restrict__ tile_ntok, int n_heads,
                    int heads_per_block, int n_splits, int n_subs) {
  const int r = blockIdx.x % ROWS;
  const int ts = blockIdx.x / ROWS;  // tile * n_subs + sub
  const int tile = ts / n_subs, sub = ts - tile * n_subs;
  const int tok = r / heads_per_block, head = sub * heads_per_block + r % heads_per_block;
  if (tok >= tile_ntok[tile] || head >= n_heads) return;
  const size_t tk = tile_tok0[tile] + tok;
  __nv_bfloat16* dst = out + tk * out_ts + (size_t)head * out_hs;
  if (tile_req[tile] < 0) {
    for (int d = threadIdx.x; d < R; d += blockDim.x) dst[d] = __float2bfloat16_rn(0.f);
    return;
  }
  const float* base = scratch + ((size_t)ts * ROWS + r) * n_splits * PART;
  // the stretches' weights once a block (the launcher allows up to MERGE_SPLITS of them)
  __shared__ float wgt_s[MERGE_SPLITS];
  __shared__ float f_s;
  if (threadIdx.x < 32) {
    float mm = -INFINITY;
    for (int s = threadIdx.x; s < n_splits; s += 32) mm = fmaxf(mm, base[(size_t)s * PART + R16]);
    mm = warp_max(mm);
    float ll = 0.f;
    for (int s = threadIdx.x; s < n_splits; s += 32) {
      const float ms = base[(size_t)s * PART + R16];
      const float wg = ms == -INFINITY ? 0.f : exp2f(ms - mm);
      wgt_s[s] = wg;
      ll += wg * base[(size_t)s * PART + R16 + 1];
    }
    ll = warp_sum(ll);
    if (threadIdx.x == 0) {
      float f = ll > 0.f ? 1.f / ll : 0.f;
      if (gate != nullptr) f *= 1.f / (1.f + __expf(-__bfloat162float(gate[tk * gate_ts + head])));
      f_s = f;
    }
  }
  __syncthreads();
  const float f = f_s;
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s) acc = fmaf(wgt_s[s], base[(size_t)s * PART + d], acc);
    dst[d] = __float2bfloat16_rn(acc * f);
  }
}

}  // namespace fg_latent

extern "C" int fg_latent_mma_rows() { return fg_latent::ROWS; }
extern "C" int fg_latent_mma_keys() { return fg_latent::KEYS; }

// Floats of scratch a launch with these numbers of tiles, head slices and stretches needs.
extern "C" long long fg_latent_mma_scratch_floats(int n_tiles, int n_heads, int n_splits) {
  using namespace fg_latent;
  const int hpb = n_heads < ROWS ? n_heads : ROWS;
  const int subs = (n_heads + hpb - 1) / hpb;
  return n_splits > 1 ? (long long)n_tiles * subs * ROWS * n_splits * PART : 0;
}

// Tiles hold ROWS / min(heads, ROWS) tokens each (the caller cuts them so).  keys_per_split is a
// multiple of the key tile; n_splits * keys_per_split covers the longest request.
extern "C" int fg_latent_attention_mma(const void* qa, long qa_ts, long qa_hs, const void* qt, long qt_ts, long qt_hs,
                                       void* out, long out_ts, long out_hs, const void* gate, long gate_ts,
                                       const void* pages, const int* block_table, int table_width, int page_size,
                                       int n_pages, const int* pos, const int* tile_req, const int* tile_tok0,
                                       const int* tile_ntok, int n_tiles, int n_heads, int rank, int rot_dim,
                                       int entry, float scale, int n_splits, int keys_per_split, float* scratch,
                                       long long scratch_floats, int* status, cudaStream_t stream) {
  using namespace fg_latent;
  if (n_tiles == 0) return 0;
  FG_CHECK_ARG(rank == R && rot_dim == ROT && entry == E,
               "fg_latent_attention_mma: library built for a latent of %d + %d (entries of %d), got %d + %d (%d)", R,
               ROT, E, rank, rot_dim, entry);
  FG_CHECK_ARG(n_splits >= 1 && n_splits <= MERGE_SPLITS && keys_per_split > 0 && keys_per_split % KEYS == 0,
               "fg_latent_attention_mma: %d stretches of %d keys", n_splits, keys_per_split);
  FG_CHECK_ARG(scratch_floats >= fg_latent_mma_scratch_floats(n_tiles, n_heads, n_splits),
               "fg_latent_attention_mma: scratch of %lld floats is too small", scratch_floats);
  FG_CHECK_ARG(qa_ts % 2 == 0 && qa_hs % 2 == 0 && qt_ts % 2 == 0 && qt_hs % 2 == 0 && out_ts % 2 == 0 &&
                   out_hs % 2 == 0 && ((uintptr_t)qa & 3) == 0 && ((uintptr_t)qt & 3) == 0 && ((uintptr_t)out & 3) == 0,
               "fg_latent_attention_mma: queries and outputs must be 4-byte aligned with even strides");
  const int hpb = n_heads < ROWS ? n_heads : ROWS;
  const int subs = (n_heads + hpb - 1) / hpb;
  constexpr size_t smem = smem_bytes();
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    FG_CHECK_ARG(e == cudaSuccess, "fg_latent_attention_mma: shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  dim3 grid(n_tiles, subs, n_splits);
  latent_attention_mma_kernel<<<grid, NTHREADS, smem, stream>>>(
      (const __nv_bfloat16*)qa, qa_ts, qa_hs, (const __nv_bfloat16*)qt, qt_ts, qt_hs, (__nv_bfloat16*)out, out_ts,
      out_hs, (const __nv_bfloat16*)gate, gate_ts, (const __nv_bfloat16*)pages, block_table, table_width, page_size,
      n_pages, pos, tile_req, tile_tok0, tile_ntok, n_heads, hpb, scale * 1.4426950408889634f, n_splits,
      keys_per_split, scratch, status);
  FG_CHECK_LAUNCH("fg_latent_attention_mma");
  if (n_splits > 1) {
    latent_merge_kernel<<<n_tiles * subs * ROWS, 128, 0, stream>>>(scratch, (__nv_bfloat16*)out, out_ts, out_hs,
                                                                   (const __nv_bfloat16*)gate, gate_ts, tile_req,
                                                                   tile_tok0, tile_ntok, n_heads, hpb, n_splits, subs);
    FG_CHECK_LAUNCH("fg_latent_merge");
  }
  return 0;
}
