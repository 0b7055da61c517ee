// MoE token movement for sm_100a: the stable expert permutation, the fused
// 1x128 e4m3 quantise-and-dispatch of activations, and the weighted combine.
//
// Row space of the grouped GEMMs. The flat list of (token, slot) entries
// i = t*k + slot is stably sorted by expert id; entry i lands at sorted position
// inv_perm[i] (perm is the inverse). Each expert's run of rows is then placed at
// a 128-aligned start in a padded row space, so that every 128-row GEMM tile
// belongs to exactly one expert:
//     dst_row[i] = pad_offsets[e] + (inv_perm[i] - offsets[e])
// tile_expert[j] names the expert of padded tile j, num_tiles[0] counts the used
// tiles. Padding rows are never written and never read back.
//
// The permutation is scan based (no atomics decide a position), so it is the
// same on every run and equal to a CPU stable sort.
#include "cab_common.cuh"

#include <cuda_fp8.h>

namespace {

constexpr int kChunk = 1024;     // entries per CTA in the count / rank kernels
constexpr int kMaxE = 256;
constexpr int kTileM = 128;

// Per-warp, per-expert population of this CTA's chunk, in shared memory:
// wc[w][e] = number of entries of expert e among warp w's 32 consecutive entries.
__device__ __forceinline__ void chunk_warp_counts(int (*wc)[kMaxE], const int* __restrict__ idx,
                                                  int n, int E, int& my_e, int& rank_in_warp,
                                                  bool& out_of_range, bool empty_ok = false) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) wc[i / E][i % E] = 0;
  __syncthreads();
  const int i = blockIdx.x * kChunk + threadIdx.x;
  my_e = i < n ? __ldg(idx + i) : -1;
  // Ids outside [0, E) are skipped and flagged; with empty_ok, -1 is the expected marker of an empty
  // slot (an unused slot of a fixed-capacity receive buffer) and is skipped without a flag.
  out_of_range = i < n && (my_e < (empty_ok ? -1 : 0) || my_e >= E);
  if (my_e < 0 || my_e >= E) my_e = -1;
  // lanes past the end all carry -1 and only match each other
  const unsigned peers = __match_any_sync(0xffffffffu, my_e);
  rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (my_e >= 0 && rank_in_warp == 0) wc[warp][my_e] = __popc(peers);
  __syncthreads();
}

// Offsets, 128-padded offsets and the tile table from per-expert populations held in shared memory
// (cnt[e], e < E <= 256), by all threads of the CTA: a warp-shuffle scan over the experts, then every
// expert writes its own run of tile_expert[].
__device__ void build_tile_table(const int* cnt, int E, int* __restrict__ offsets, int* __restrict__ pad_offsets,
                                 int* __restrict__ tile_expert, int* __restrict__ num_tiles, int max_tiles,
                                 int* __restrict__ status, int* scan_sm /* 2 * 8 ints */) {
  __shared__ int total_tiles;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = tid < E ? cnt[tid] : 0;
  const int nt = (c + kTileM - 1) / kTileM;
  int inc_c = c, inc_t = nt;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, inc_c, off), b = __shfl_up_sync(0xffffffffu, inc_t, off);
    if (lane >= off) { inc_c += a; inc_t += b; }
  }
  if (warp < 8 && lane == 31) { scan_sm[warp] = inc_c; scan_sm[8 + warp] = inc_t; }
  __syncthreads();
  int base_c = 0, base_t = 0;
  for (int w = 0; w < warp && w < 8; ++w) { base_c += scan_sm[w]; base_t += scan_sm[8 + w]; }
  const int off_c = base_c + inc_c - c, off_t = base_t + inc_t - nt;     // exclusive
  if (tid < E) {
    offsets[tid] = off_c;
    pad_offsets[tid] = off_t * kTileM;
    for (int j = 0; j < nt; ++j)
      if (off_t + j < max_tiles) tile_expert[off_t + j] = tid;
  }
  if (tid == E - 1) {
    const int tiles = off_t + nt;
    offsets[E] = off_c + c;
    pad_offsets[E] = tiles * kTileM;
    if (tiles > max_tiles && status) atomicExch(status, 2);
    num_tiles[0] = min(tiles, max_tiles);
    total_tiles = min(tiles, max_tiles);
  }
  __syncthreads();
  for (int j = total_tiles + tid; j < max_tiles; j += blockDim.x) tile_expert[j] = -1;
}

// Kernel 1: per-chunk expert counts; the last CTA to finish turns them into
// chunk bases, expert offsets, padded offsets and the tile table.
__global__ void __launch_bounds__(kChunk)
moe_count_scan_kernel(const int* __restrict__ idx, int n, int E, int nchunks,
                      int* __restrict__ chunk_cnt,   // [nchunks][E], becomes exclusive chunk bases
                      unsigned* __restrict__ done_counter,
                      int* __restrict__ counts, int* __restrict__ offsets,
                      int* __restrict__ pad_offsets, int* __restrict__ tile_expert,
                      int* __restrict__ num_tiles, int max_tiles, int* __restrict__ status, bool empty_ok) {
  __shared__ int wc[32][kMaxE];
  __shared__ bool is_last;
  int my_e, rank;
  bool bad;
  chunk_warp_counts(wc, idx, n, E, my_e, rank, bad, empty_ok);
  if (bad && status) atomicExch(status, 1);   // expert id out of range: flagged, entry ignored
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int c = 0;
#pragma unroll 8
    for (int w = 0; w < 32; ++w) c += wc[w][e];
    chunk_cnt[(size_t)blockIdx.x * E + e] = c;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(done_counter, 1u) == (unsigned)nchunks - 1u);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // exclusive scan over chunks: a warp per expert, 32 chunks per shuffle scan
  {
    const int lane = threadIdx.x & 31;
    for (int e = threadIdx.x >> 5; e < E; e += kChunk / 32) {
      int run = 0;
      for (int c0 = 0; c0 < nchunks; c0 += 32) {
        const int c = c0 + lane;
        const int v = c < nchunks ? __ldcg(chunk_cnt + (size_t)c * E + e) : 0;
        int inc = v;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int a = __shfl_up_sync(0xffffffffu, inc, off);
          if (lane >= off) inc += a;
        }
        if (c < nchunks) chunk_cnt[(size_t)c * E + e] = run + inc - v;
        run += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (lane == 0) { counts[e] = run; wc[0][e] = run; }
    }
  }
  __syncthreads();
  build_tile_table(wc[0], E, offsets, pad_offsets, tile_expert, num_tiles, max_tiles, status, &wc[1][0]);
  if (threadIdx.x == 0) *done_counter = 0;   // ready for the next call
}

// Kernel 2: position of every entry.
__global__ void __launch_bounds__(kChunk)
moe_rank_kernel(const int* __restrict__ idx, int n, int E, const int* __restrict__ chunk_base,
                const int* __restrict__ offsets, const int* __restrict__ pad_offsets,
                int* __restrict__ perm, int* __restrict__ inv_perm, int* __restrict__ dst_row, int max_rows) {
  __shared__ int wc[32][kMaxE];
  int my_e, rank;
  bool bad;
  chunk_warp_counts(wc, idx, n, E, my_e, rank, bad);
  // exclusive scan over the 32 warps, one thread per expert
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
#pragma unroll 8
    for (int w = 0; w < 32; ++w) { const int v = wc[w][e]; wc[w][e] = run; run += v; }
  }
  __syncthreads();
  const int i = blockIdx.x * kChunk + threadIdx.x;
  if (i >= n) return;
  if (my_e >= 0) {
    const int within = __ldg(chunk_base + (size_t)blockIdx.x * E + my_e) + wc[threadIdx.x >> 5][my_e] + rank;
    const int pos = __ldg(offsets + my_e) + within;
    inv_perm[i] = pos;
    perm[pos] = i;
    // rows past the tile table's capacity (flagged as overflow by the count kernel) belong to no tile
    const int row = __ldg(pad_offsets + my_e) + within;
    dst_row[i] = row < max_rows ? row : -1;
  } else {
    // a skipped entry has no row: the quantise-dispatch and combine kernels pass over negative rows
    inv_perm[i] = -1;
    dst_row[i] = -1;
  }
  // sorted positions past the last valid entry name no entry
  if (i >= __ldg(offsets + E)) perm[i] = -1;
}

// ------------------------------------------------------------------ quantise + dispatch
// amax floor and the e4m3 maximum of the 1x128 quantisation rule.
constexpr float kAmaxFloor = 1e-4f;
constexpr float kFp8Max = 448.f;

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

// One warp per token. Per pass the warp covers 256 columns: a lane reads 8 bf16
// (16 bytes); a 128-column quantisation block is a half-warp. The quantised row
// is written to every destination row of the token (k of them, or row t itself
// when dst_row is null), scales go to the transposed table sc_t[block][row].
// ROW_MAJOR_SCALES: scales go to sc[row * (H/128) + block] instead (the layout a row travels in).
template <bool ROW_MAJOR_SCALES>
__global__ void __launch_bounds__(256)
moe_quant_dispatch_kernel(const __nv_bfloat16* __restrict__ x, int T, int H, int k,
                          const int* __restrict__ dst_row, uint8_t* __restrict__ a_q,
                          float* __restrict__ sc_t, int ld_rows) {
  // a warp per (token, 1024-column segment): long rows are shared by several warps
  const int lane = threadIdx.x & 31;
  const int segs = (H + 1023) >> 10;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)T * segs) return;
  const int t = (int)(w / segs);
  const int c0 = (int)(w - (long long)t * segs) << 10;
  int my_dst = t;
  if (dst_row) my_dst = lane < k ? __ldg(dst_row + (size_t)t * k + lane) : -1;
  const int ndst = dst_row ? k : 1;
  const uint4* xrow = reinterpret_cast<const uint4*>(x + (size_t)t * H);
  // the four 16-byte loads of a lane are issued before the first is used
  {
    uint4 raw4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int col = c0 + u * 256 + lane * 8;
      raw4[u] = col < H ? __ldg(xrow + (col >> 3)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int col = c0 + u * 256 + lane * 8;
      const bool live = col < H;
      if (c0 + u * 256 >= H) break;                      // warp-uniform: nothing left of the row
      const uint4 raw = raw4[u];
      float v[8] = {cab::bf16_lo(raw.x), cab::bf16_hi(raw.x), cab::bf16_lo(raw.y), cab::bf16_hi(raw.y),
                    cab::bf16_lo(raw.z), cab::bf16_hi(raw.z), cab::bf16_lo(raw.w), cab::bf16_hi(raw.w)};
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
      const float scale = __fdiv_rn(fmaxf(amax, kAmaxFloor), kFp8Max);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __fdiv_rn(v[j], scale);
      const uint2 q = make_uint2(pack4_e4m3(v[0], v[1], v[2], v[3]), pack4_e4m3(v[4], v[5], v[6], v[7]));
      for (int s = 0; s < ndst; ++s) {
        const int row = dst_row ? __shfl_sync(0xffffffffu, my_dst, s) : t;
        if (live && row >= 0) {
          *reinterpret_cast<uint2*>(a_q + (size_t)row * H + col) = q;
          if ((lane & 15) == 0) {
            if (ROW_MAJOR_SCALES) sc_t[(size_t)row * (H >> 7) + (col >> 7)] = scale;
            else sc_t[(size_t)(col >> 7) * ld_rows + row] = scale;
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------ combine
// out[t] = sum over slots (ascending) of w[t,slot] * y[dst_row[t*k+slot]] (+ extra[t]),
// fp32 accumulate, bf16 result; slots with a negative row are skipped. One CTA per token, 16-byte accesses.
template <int BATCH>
__global__ void __launch_bounds__(256)
moe_combine_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ y,
                   const int* __restrict__ dst_row, const float* __restrict__ w,
                   const __nv_bfloat16* __restrict__ extra, int T, int H, int k) {
  const int t = blockIdx.x;
  __shared__ int rows[32];
  __shared__ float wts[32];
  if (threadIdx.x < k) {
    rows[threadIdx.x] = __ldg(dst_row + (size_t)t * k + threadIdx.x);
    wts[threadIdx.x] = __ldg(w + (size_t)t * k + threadIdx.x);
  }
  __syncthreads();
  for (int col = threadIdx.x * 8; col < H; col += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // Slots in batches of BATCH: the batch's row loads are issued together, then added in ascending slot
    // order; an empty slot (a copy whose experts use fewer than k slots on this rank) contributes 0 * 0.
    // (BATCH follows k: registers spent on a batch that k cannot fill would only cost resident CTAs.)
    for (int s0 = 0; s0 < k; s0 += BATCH) {
      uint4 raw[BATCH];
      float ws[BATCH];
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int s = s0 + u;
        const bool live = s < k && rows[s] >= 0;
        raw[u] = live ? __ldcs(reinterpret_cast<const uint4*>(y + (size_t)rows[s] * H + col)) : make_uint4(0u, 0u, 0u, 0u);
        ws[u] = live ? wts[s] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        acc[0] = fmaf(ws[u], cab::bf16_lo(raw[u].x), acc[0]); acc[1] = fmaf(ws[u], cab::bf16_hi(raw[u].x), acc[1]);
        acc[2] = fmaf(ws[u], cab::bf16_lo(raw[u].y), acc[2]); acc[3] = fmaf(ws[u], cab::bf16_hi(raw[u].y), acc[3]);
        acc[4] = fmaf(ws[u], cab::bf16_lo(raw[u].z), acc[4]); acc[5] = fmaf(ws[u], cab::bf16_hi(raw[u].z), acc[5]);
        acc[6] = fmaf(ws[u], cab::bf16_lo(raw[u].w), acc[6]); acc[7] = fmaf(ws[u], cab::bf16_hi(raw[u].w), acc[7]);
      }
    }
    if (extra) {
      const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(extra + (size_t)t * H + col));
      acc[0] += cab::bf16_lo(raw.x); acc[1] += cab::bf16_hi(raw.x);
      acc[2] += cab::bf16_lo(raw.y); acc[3] += cab::bf16_hi(raw.y);
      acc[4] += cab::bf16_lo(raw.z); acc[5] += cab::bf16_hi(raw.z);
      acc[6] += cab::bf16_lo(raw.w); acc[7] += cab::bf16_hi(raw.w);
    }
    __nv_bfloat162 p0 = __floats2bfloat162_rn(acc[0], acc[1]), p1 = __floats2bfloat162_rn(acc[2], acc[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[4], acc[5]), p3 = __floats2bfloat162_rn(acc[6], acc[7]);
    uint4 o;
    o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
    o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
    *reinterpret_cast<uint4*>(out + (size_t)t * H + col) = o;
  }
}

// ------------------------------------------------------------------ expert-parallel row movement
// Received rows (quantised bytes + row-major scales, in arrival order) -> the padded row space of the
// local grouped GEMMs: a_q[dst_row[i]] = rows[i], scales transposed on the way.
__global__ void __launch_bounds__(256)
moe_scatter_rows_kernel(uint8_t* __restrict__ a_q, float* __restrict__ sc_t, const uint8_t* __restrict__ rows,
                        const float* __restrict__ scales, const int* __restrict__ dst_row, int n, int H, int ld_rows) {
  const int i = blockIdx.x;
  const int d = __ldg(dst_row + i);
  if (d < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(rows + (size_t)i * H);
  uint4* dst = reinterpret_cast<uint4*>(a_q + (size_t)d * H);
  for (int c = threadIdx.x; c < H / 16; c += blockDim.x) dst[c] = __ldcs(src + c);
  for (int b = threadIdx.x; b < H / 128; b += blockDim.x) sc_t[(size_t)b * ld_rows + d] = __ldg(scales + (size_t)i * (H / 128) + b);
}

// out[i, :] = y[src_row[i], :] (bf16 rows of H elements): the way back, before the return exchange.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(uint4* __restrict__ out, const uint4* __restrict__ y, const int* __restrict__ src_row, int H) {
  const int i = blockIdx.x;
  const int s = __ldg(src_row + i);
  const int n16 = H / 8;
  for (int c = threadIdx.x; c < n16; c += blockDim.x)
    out[(size_t)i * n16 + c] = s >= 0 ? __ldcs(y + (size_t)s * n16 + c) : make_uint4(0, 0, 0, 0);
}

// Tile table of the local experts from their populations (what moe_count_scan_kernel derives from
// the routing when everything is local).
__global__ void __launch_bounds__(256)
moe_tiles_from_counts_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                             int* __restrict__ pad_offsets, int* __restrict__ tile_expert,
                             int* __restrict__ num_tiles, int max_tiles) {
  __shared__ int cnt[kMaxE];
  __shared__ int scan_sm[16];
  if (threadIdx.x < E) cnt[threadIdx.x] = counts[threadIdx.x];
  __syncthreads();
  build_tile_table(cnt, E, offsets, pad_offsets, tile_expert, num_tiles, max_tiles, nullptr, scan_sm);
}

}  // namespace

extern "C" size_t moe_permute_scratch_bytes(int T, int k, int E) {
  const long long n = (long long)T * k;
  const long long nchunks = n <= 0 ? 1 : (n + kChunk - 1) / kChunk;   // the launcher runs one chunk when empty
  return (size_t)(nchunks * E + 2) * sizeof(int);
}

extern "C" int moe_permute_max_tiles(int T, int k, int E) {
  // every expert can waste at most one partial tile
  const long long n = (long long)T * k;
  return (int)(n / kTileM + E);
}

extern "C" int moe_permute_launcher(const int* topk_idx, int T, int k, int E, int* counts,
                                    int* offsets, int* pad_offsets, int* perm, int* inv_perm,
                                    int* dst_row, int* tile_expert, int* num_tiles, int max_tiles,
                                    void* scratch, int config, cudaStream_t stream) {
  if (!counts || !offsets || !pad_offsets || !tile_expert || !num_tiles || !scratch)
    return CAB_ERR_BAD_ARGUMENT;
  if (T < 0 || k <= 0 || E <= 0 || E > kMaxE || max_tiles <= 0) return CAB_ERR_BAD_ARGUMENT;
  const long long n = (long long)T * k;
  if (n > 0 && (!topk_idx || !perm || !inv_perm || !dst_row)) return CAB_ERR_BAD_ARGUMENT;
  if (n > (1LL << 30)) return CAB_ERR_TOO_LARGE;
  const int nchunks = n == 0 ? 1 : (int)((n + kChunk - 1) / kChunk);
  int* chunk_cnt = static_cast<int*>(scratch);
  unsigned* done = reinterpret_cast<unsigned*>(chunk_cnt + (size_t)nchunks * E);
  int* status = chunk_cnt + (size_t)nchunks * E + 1;
  if (cudaMemsetAsync(done, 0, 2 * sizeof(int), stream) != cudaSuccess) return CAB_ERR_LAUNCH;
  moe_count_scan_kernel<<<nchunks, kChunk, 0, stream>>>(topk_idx, (int)n, E, nchunks, chunk_cnt, done,
                                                        counts, offsets, pad_offsets, tile_expert,
                                                        num_tiles, max_tiles, status, (config & 1) != 0);
  if (n > 0)
    moe_rank_kernel<<<nchunks, kChunk, 0, stream>>>(topk_idx, (int)n, E, chunk_cnt, offsets,
                                                    pad_offsets, perm, inv_perm, dst_row,
                                                    max_tiles > (1 << 24) ? 0x7fffffff : max_tiles * kTileM);
  return cab::launch_status();
}

static unsigned quant_dispatch_grid(int T, int H) {   // eight warps per CTA, a warp per (token, 1024 columns)
  const long long warps = (long long)T * ((H + 1023) >> 10);
  return (unsigned)((warps + 7) / 8);
}

extern "C" int moe_quant_dispatch_launcher(cab_e4m3* a_q, float* scales_t, const cab_bf16* x,
                                           const int* dst_row, int T, int H, int k, int ld_rows,
                                           int config, cudaStream_t stream) {
  (void)config;
  if (T == 0) return CAB_OK;
  if (!a_q || !scales_t || !x) return CAB_ERR_BAD_ARGUMENT;
  if (T < 0 || H <= 0 || H % 128 != 0 || k <= 0 || k > 32 || ld_rows <= 0) return CAB_ERR_BAD_ARGUMENT;
  if (!cab::aligned_to(a_q, 16) || !cab::aligned_to(x, 16)) return CAB_ERR_MISALIGNED;
  moe_quant_dispatch_kernel<false><<<quant_dispatch_grid(T, H), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), T, H, k, dst_row, a_q, scales_t, ld_rows);
  return cab::launch_status();
}

extern "C" int moe_quant_rows_launcher(cab_e4m3* rows_q, float* scales, const cab_bf16* x, const int* dst_row,
                                       int T, int H, int k, int config, cudaStream_t stream) {
  (void)config;
  if (T == 0) return CAB_OK;
  if (!rows_q || !scales || !x) return CAB_ERR_BAD_ARGUMENT;
  if (T < 0 || H <= 0 || H % 128 != 0 || k <= 0 || k > 32) return CAB_ERR_BAD_ARGUMENT;
  if (!cab::aligned_to(rows_q, 16) || !cab::aligned_to(x, 16)) return CAB_ERR_MISALIGNED;
  moe_quant_dispatch_kernel<true><<<quant_dispatch_grid(T, H), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), T, H, k, dst_row, rows_q, scales, 0);
  return cab::launch_status();
}

extern "C" int moe_combine_launcher(cab_bf16* out, const cab_bf16* y, const int* dst_row,
                                    const float* weights, const cab_bf16* extra, int T, int H, int k,
                                    int config, cudaStream_t stream) {
  (void)config;
  if (T == 0) return CAB_OK;
  if (!out || !y || !dst_row || !weights) return CAB_ERR_BAD_ARGUMENT;
  if (T < 0 || H <= 0 || H % 8 != 0 || k <= 0 || k > 32) return CAB_ERR_BAD_ARGUMENT;
  if (!cab::aligned_to(out, 16) || !cab::aligned_to(y, 16) || (extra && !cab::aligned_to(extra, 16)))
    return CAB_ERR_MISALIGNED;
  const int threads = cab::row_walk_threads(H / 8);
  auto* o = reinterpret_cast<__nv_bfloat16*>(out);
  auto* yy = reinterpret_cast<const __nv_bfloat16*>(y);
  auto* ex = reinterpret_cast<const __nv_bfloat16*>(extra);
  if (k <= 2) moe_combine_kernel<2><<<T, threads, 0, stream>>>(o, yy, dst_row, weights, ex, T, H, k);
  else if (k <= 4) moe_combine_kernel<4><<<T, threads, 0, stream>>>(o, yy, dst_row, weights, ex, T, H, k);
  else moe_combine_kernel<8><<<T, threads, 0, stream>>>(o, yy, dst_row, weights, ex, T, H, k);
  return cab::launch_status();
}

extern "C" int moe_scatter_rows_launcher(cab_e4m3* a_q, float* scales_t, const cab_e4m3* rows, const float* scales,
                                         const int* dst_row, int n, int H, int ld_rows, int config,
                                         cudaStream_t stream) {
  (void)config;
  if (n == 0) return CAB_OK;
  if (!a_q || !scales_t || !rows || !scales || !dst_row) return CAB_ERR_BAD_ARGUMENT;
  if (n < 0 || H <= 0 || H % 128 != 0 || ld_rows <= 0) return CAB_ERR_BAD_ARGUMENT;
  if (!cab::aligned_to(a_q, 16) || !cab::aligned_to(rows, 16)) return CAB_ERR_MISALIGNED;
  moe_scatter_rows_kernel<<<n, 256, 0, stream>>>(a_q, scales_t, rows, scales, dst_row, n, H, ld_rows);
  return cab::launch_status();
}

extern "C" int moe_gather_rows_launcher(cab_bf16* out, const cab_bf16* y, const int* src_row, int n, int H,
                                        int config, cudaStream_t stream) {
  (void)config;
  if (n == 0) return CAB_OK;
  if (!out || !y || !src_row || n < 0 || H <= 0 || H % 8 != 0) return CAB_ERR_BAD_ARGUMENT;
  if (!cab::aligned_to(out, 16) || !cab::aligned_to(y, 16)) return CAB_ERR_MISALIGNED;
  moe_gather_rows_kernel<<<n, 256, 0, stream>>>(reinterpret_cast<uint4*>(out), reinterpret_cast<const uint4*>(y),
                                                src_row, H);
  return cab::launch_status();
}

extern "C" int moe_tiles_from_counts_launcher(const int* counts, int E, int* offsets, int* pad_offsets,
                                              int* tile_expert, int* num_tiles, int max_tiles, int config,
                                              cudaStream_t stream) {
  (void)config;
  if (!counts || !offsets || !pad_offsets || !tile_expert || !num_tiles || E <= 0 || max_tiles <= 0)
    return CAB_ERR_BAD_ARGUMENT;
  if (E > kMaxE) return CAB_ERR_TOO_LARGE;
  moe_tiles_from_counts_kernel<<<1, 256, 0, stream>>>(counts, E, offsets, pad_offsets, tile_expert, num_tiles, max_tiles);
  return cab::launch_status();
}
