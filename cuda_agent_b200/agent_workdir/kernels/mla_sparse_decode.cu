// Top-k sparse MLA decode attention for sm_100a (absorbed latent attention, one query
// token per sequence): out[b,h,:] = softmax_j(q[b,h,:] . kv[b, idx[b,j], :] * scale) . kv[b, idx[b,j], :512]
// over the valid entries of idx (0 <= idx < seq_len[b]).
//
// Two kernels. Head groups of 128 run on pairs of CTAs that split the 576 columns between them
// (mla_sparse_decode_pair_kernel, described further down); other head counts (multiples of 64), and
// config 1, use the kernel described here: one CTA handles 64 query heads of one sequence and one
// contiguous range ("split") of the selected rows, 64 rows at a time:
//   producer warps (4)  gather the 64 selected cache rows (1152 B each) into shared memory with
//                       16-byte cp.async copies, laid out as nine 64-row x 128-byte tiles in the
//                       128-byte swizzle the tensor core reads; two stages
//   MMA warp (1 thread) S = Q . K^T   : tcgen05.mma kind::f16, M=64 N=64, 36 steps of K=16
//                       O += P . V    : V is the first 512 columns of the same tile read as an
//                                       MN-major operand, two M=64 N=256 accumulators that share
//                                       256 tensor-memory columns (lanes 0-15 / 16-31 of each quadrant)
//                       issue order follows readiness: Q.K^T of block j+1 overlaps the softmax of
//                       block j when its rows have landed, P.V of block j releases its stage
//   softmax warps (4)   read S from tensor memory (one head per thread, lanes 0-15 of each warp),
//                       scale, mask invalid entries, online softmax in the exp2 domain with a lazy
//                       reference maximum (O is rescaled in tensor memory only when the running
//                       maximum grows by more than 2^8), write P as bf16 into shared memory
// All mbarrier waits are bounded. With nsplit > 1 the CTAs write unnormalised fp32 partials
// plus (reference maximum, sum) and a second kernel merges them.
#include "cab_common.cuh"
#include "sm100_primitives.cuh"

#include <cstring>
#include <mutex>

namespace {

constexpr int kDqk = 576, kDv = 512;
constexpr int kHeads = 64;                 // heads per CTA (UMMA M)
constexpr int kTok = 64;                   // selected rows per block (UMMA N of QK, K of PV)
constexpr int kChunks = kDqk / 64;         // 9 tiles of 64 columns
constexpr int kChunkBytes = 64 * 128;      // 64 rows x 128 bytes
constexpr int kTileBytes = kChunks * kChunkBytes;   // 73728: Q (64 heads) or one K stage (64 rows)
constexpr int kPBytes = kHeads * 128;      // P: 64 heads x 64 tokens bf16
constexpr int kProducerThreads = 128;
constexpr int kThreads = 9 * 32;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 128;
constexpr float kRescaleThreshold = 8.f;   // log2 units

struct __align__(16) Control {
  uint64_t kv_full[2], kv_empty[2], s_full[2], s_empty[2], p_full, p_empty, o_done;
  uint32_t tmem_base;
  int abort_flag;
  unsigned char valid[2][kTok];
};
constexpr int kSmemBytes = 3 * kTileBytes + kPBytes + (int)sizeof(Control) + 1024;

struct MlaParams {
  const __nv_bfloat16* q;      // [B, Sq, Hh, 576]
  const __nv_bfloat16* kv;     // [B, S, 576]
  const int* seq_len;          // [B, Sq]
  const int* idx;              // [B, Sq, topk]
  __nv_bfloat16* out;          // [B, Sq, Hh, 512]                (nsplit == 1)
  float* part_o;               // [B*Sq, nsplit, Hh, 512] unnormalised (nsplit > 1)
  float* part_ml;              // [B*Sq, nsplit, Hh, 2]  (reference max in log2 units, sum)
  int Hh, S, topk, nsplit, Sq; // Sq query tokens per sequence share its cache rows
  float scale_log2;            // softmax scale * log2(e)
  int* status;
};

enum { kWaitKvFull = 201, kWaitKvEmpty = 202, kWaitSFull = 203, kWaitSEmpty = 204, kWaitPFull = 205,
       kWaitPEmpty = 206, kWaitODone = 207 };

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// 16-column forms of the tensor-memory load and store (thread i: lane quadrant base + i, columns [col, col+16)).
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Operand descriptor for 128-byte-swizzled tiles; offsets in bytes.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((smem_addr >> 4) & 0x3fff) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// Copies `rows` x 576 bf16 (16-byte pieces, coalesced per row) into the nine swizzled tiles at `dst`.
// `src_row(r)` yields the global pointer of row r.
template <typename RowPtr>
__device__ __forceinline__ void gather_tile(uint32_t dst, int tid, int nthreads, RowPtr src_row) {
  for (int id = tid; id < kTok * 72; id += nthreads) {
    const int r = id / 72, c16 = id - r * 72;
    const int chunk = c16 >> 3, within = c16 & 7;
    cp_async_16(dst + chunk * kChunkBytes + r * 128 + ((within ^ (r & 7)) << 4), src_row(r) + c16 * 8);
  }
}

__global__ void __launch_bounds__(kThreads, 1) mla_sparse_decode_kernel(const MlaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_tile = base;
  uint8_t* kv_tile = base + kTileBytes;              // two stages
  uint8_t* p_tile = base + 3 * kTileBytes;
  Control& ctl = *reinterpret_cast<Control*>(p_tile + kPBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head0 = blockIdx.x * kHeads, split = blockIdx.y, b = blockIdx.z;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      sm100::mbar_init(&ctl.kv_full[s], kProducerThreads);
      sm100::mbar_init(&ctl.kv_empty[s], 1);
      sm100::mbar_init(&ctl.s_full[s], 1);
      sm100::mbar_init(&ctl.s_empty[s], 4);
    }
    sm100::mbar_init(&ctl.p_full, 4);
    sm100::mbar_init(&ctl.p_empty, 1);
    sm100::mbar_init(&ctl.o_done, 1);
    ctl.abort_flag = 0;
    sm100::mbar_fence_init();
  }
  if (warp == 4) {
    sm100::tmem_alloc(&ctl.tmem_base, kTmemCols);
    sm100::tmem_relinquish();
  }
  // Q tile: 64 heads x 576, every thread helps
  {
    const __nv_bfloat16* qb = p.q + ((size_t)b * p.Hh + head0) * kDqk;
    gather_tile(sm100::smem_u32(q_tile), threadIdx.x, kThreads,
                [&](int r) { return qb + (size_t)r * kDqk; });
    cp_async_commit();
    cp_async_wait<0>();
    sm100::fence_proxy_async();
  }
  sm100::tc_fence_before_sync();
  __syncthreads();
  sm100::tc_fence_after_sync();
  const uint32_t tmem_base = ctl.tmem_base;
  volatile int* abort_flag = &ctl.abort_flag;

  const int blocks_total = (p.topk + kTok - 1) / kTok;
  const int per_split = (blocks_total + p.nsplit - 1) / p.nsplit;
  const int j0 = split * per_split;
  const int nb = max(0, min(blocks_total, j0 + per_split) - j0);
  const int len = min(__ldg(p.seq_len + b), p.S);   // a length past the cache's extent never reaches a row outside it

  if (warp >= 5) {
    // ---------------------------------------------------------------- producers
    const int ptid = threadIdx.x - 5 * 32;
    const int* idx_b = p.idx + (size_t)b * p.topk;
    const __nv_bfloat16* kv_b = p.kv + (size_t)(b / p.Sq) * p.S * kDqk;   // b counts (sequence, query token) pairs
    // Iteration j: publish block j-1 as soon as it has landed (nothing newer is in flight yet), then
    // wait for the stage of block j to be released by P.V of block j-2 and start its copies. Block j is
    // in flight while block j-1 is computed.
    // Geometry of this lane's 36 pieces (which of the warp's 16 rows, where in the tile, which 16 bytes
    // of the cache row) does not depend on the block.
    const int pw = ptid >> 5;
    int piece_row[36];
    uint32_t piece_dst[36];
    int piece_src[36];
#pragma unroll
    for (int it = 0; it < 36; ++it) {
      const int piece = it * 32 + lane;
      const int rl = piece / 72, c16 = piece - rl * 72;
      const int r = pw * 16 + rl;
      piece_row[it] = rl;
      piece_dst[it] = (c16 >> 3) * kChunkBytes + r * 128 + (((c16 & 7) ^ (r & 7)) << 4);
      piece_src[it] = c16 * 8;
    }
    for (int j = 0; j <= nb; ++j) {
      if (j >= 1) {
        cp_async_wait<0>();
        sm100::fence_proxy_async();
        sm100::mbar_arrive(&ctl.kv_full[(j - 1) & 1]);
      }
      if (j == nb) break;
      const int st = j & 1;
      if (j >= 2 && !sm100::mbar_wait_relaxed(&ctl.kv_empty[st], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kWaitKvEmpty))
        break;
      // Warp w of the producers owns rows 16w..16w+15 of the block: lane l fetches the cache row
      // number of row 16w + (l & 15) once, the 1152 sixteen-byte pieces of the 16 rows are spread over
      // the lanes (36 each) and every piece learns its row by shuffle.
      const int my_i = (j0 + j) * kTok + pw * 16 + (lane & 15);
      const int my_t = my_i < p.topk ? __ldg(idx_b + my_i) : -1;
      const bool my_ok = my_t >= 0 && my_t < len;
      if (lane < 16) ctl.valid[st][pw * 16 + lane] = my_ok ? 1 : 0;
      // an invalid entry copies row 0: finite data that the mask multiplies by zero
      const int my_row = my_ok ? my_t : 0;
      const uint32_t dst = sm100::smem_u32(kv_tile + st * kTileBytes);
#pragma unroll
      for (int it = 0; it < 36; ++it) {
        const int t = __shfl_sync(0xffffffffu, my_row, piece_row[it]);
        cp_async_16(dst + piece_dst[it], kv_b + (size_t)t * kDqk + piece_src[it]);
      }
      cp_async_commit();
    }
  } else if (warp == 4) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = sm100::umma_idesc(1 /* bf16 */, kHeads, kTok);
      constexpr uint32_t idesc_pv = sm100::umma_idesc(1, kHeads, 256) | (1u << 16);   // B is MN-major
      const uint32_t q_addr = sm100::smem_u32(q_tile), p_addr = sm100::smem_u32(p_tile);
      bool ok = true;
      auto issue_pv = [&](int i) {
        const int st = i & 1;
        if (!sm100::mbar_wait(&ctl.p_full, i & 1, abort_flag, p.status, kWaitPFull)) { ok = false; return; }
        sm100::tc_fence_after_sync();
        const uint32_t v_addr = sm100::smem_u32(kv_tile + st * kTileBytes);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const uint32_t d = tmem_base + kColO + (half ? (16u << 16) : 0u);
          const uint64_t a = umma_desc_sw128(p_addr, 16, 1024);
          const uint64_t bd = umma_desc_sw128(v_addr + half * 4 * kChunkBytes, kChunkBytes, 1024);
#pragma unroll
          for (int k4 = 0; k4 < kTok / 16; ++k4)   // 16 tokens per step: 32 B along P rows, 2 KiB down V
            sm100::umma_f16(d, a + 2 * k4, bd + (uint64_t)k4 * (2048 >> 4), idesc_pv, (i > 0 || k4 > 0) ? 1u : 0u);
        }
        sm100::umma_commit(&ctl.kv_empty[st]);
        sm100::umma_commit(&ctl.p_empty);
      };
      // Issue order is decided by what is ready: Q.K^T of the next block as soon as its rows have landed
      // (at most one block ahead of P.V, so that the softmax of block j overlaps Q.K^T of block j+1),
      // otherwise P.V of the oldest block whose P is written. The stage of block j is released by its
      // P.V, and the gather of block j+2 goes into it.
      int next_qk = 0, next_pv = 0;
      const long long t_start = clock64();
      uint32_t spin = 0;
      while (next_pv < nb && ok) {
        bool issued = false;
        if (next_qk < nb && next_qk <= next_pv + 1) {
          const int j = next_qk, st = j & 1;
          const uint32_t ph = (j >> 1) & 1;
          if (sm100::mbar_try_wait(&ctl.kv_full[st], ph) && sm100::mbar_try_wait(&ctl.s_empty[st], ph ^ 1)) {
            sm100::tc_fence_after_sync();
            const uint32_t k_addr = sm100::smem_u32(kv_tile + st * kTileBytes);
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
              const uint64_t a = umma_desc_sw128(q_addr + c * kChunkBytes, 16, 1024);
              const uint64_t bd = umma_desc_sw128(k_addr + c * kChunkBytes, 16, 1024);
#pragma unroll
              for (int k4 = 0; k4 < 4; ++k4)
                sm100::umma_f16(tmem_base + kColS + st * kTok, a + 2 * k4, bd + 2 * k4, idesc_qk, (c > 0 || k4 > 0) ? 1u : 0u);
            }
            sm100::umma_commit(&ctl.s_full[st]);
            ++next_qk;
            issued = true;
          }
        }
        if (!issued && next_pv < next_qk && sm100::mbar_try_wait(&ctl.p_full, next_pv & 1)) {
          issue_pv(next_pv);
          ++next_pv;
          issued = true;
        }
        if (issued) { spin = 0; continue; }
        if ((++spin & 0x3ff) == 0) {
          if (*abort_flag) { ok = false; break; }
          if (clock64() - t_start > (long long)(nb + 2) * sm100::kWaitLimitCycles) {
            *abort_flag = 1;
            if (p.status) atomicCAS(p.status, 0, kWaitKvFull);
            ok = false;
          }
        }
      }
      if (ok) sm100::umma_commit(&ctl.o_done);
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax + epilogue (warps 0..3)
    const bool row_ok = lane < 16;                 // M=64 accumulators live in lanes 0-15 of each quadrant
    const int head = head0 + warp * 16 + (lane & 15);
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < nb; ++j) {
      const int st = j & 1;
      int got = 1;
      if (lane == 0) got = sm100::mbar_wait(&ctl.s_full[st], (j >> 1) & 1, abort_flag, p.status, kWaitSFull);
      if (!__shfl_sync(0xffffffffu, got, 0)) { ok = false; break; }
      sm100::tc_fence_after_sync();
      uint32_t t0[32], t1[32];
      sm100::tmem_ld_32x32(lane_base + kColS + st * kTok, t0);
      sm100::tmem_ld_32x32(lane_base + kColS + st * kTok + 32, t1);
      sm100::tmem_ld_wait();
      sm100::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&ctl.s_empty[st]);

      // validity of the block's 64 entries as two ballots
      const unsigned v_lo = __ballot_sync(0xffffffffu, ctl.valid[st][lane] != 0);
      const unsigned v_hi = __ballot_sync(0xffffffffu, ctl.valid[st][lane + 32] != 0);
      // masked raw scores stay in the registers the tensor-memory load filled; the softmax scale is
      // folded into the exponent: p = exp2(raw * scale_log2 - m)
      float m_raw = -INFINITY;
#pragma unroll
      for (int i = 0; i < kTok; ++i) {
        uint32_t& slot = i < 32 ? t0[i] : t1[i - 32];
        const bool live = row_ok && (((i < 32 ? v_lo : v_hi) >> (i & 31)) & 1u);
        const float raw = live ? __uint_as_float(slot) : -INFINITY;
        slot = __float_as_uint(raw);
        m_raw = fmaxf(m_raw, raw);
      }
      const float m_blk = m_raw * p.scale_log2;            // scale > 0: the maximum commutes with it
      // lazy reference maximum: move it only on the first non-empty block or on a jump > 2^8
      float factor = 1.f;
      if (m_blk > -INFINITY) {
        if (m_ref == -INFINITY) {
          m_ref = m_blk;
        } else if (m_blk > m_ref + kRescaleThreshold) {
          factor = exp2f(m_ref - m_blk);
          m_ref = m_blk;
        }
      }
      const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;   // exp2(-inf) = 0 for masked entries
      float psum = 0.f;
      uint32_t packed[kTok / 2];
#pragma unroll
      for (int i = 0; i < kTok; i += 2) {
        const float r0 = __uint_as_float(i < 32 ? t0[i] : t1[i - 32]);
        const float r1 = __uint_as_float(i + 1 < 32 ? t0[i + 1] : t1[i + 1 - 32]);
        const float p0 = exp2f(fmaf(r0, p.scale_log2, neg_m)), p1 = exp2f(fmaf(r1, p.scale_log2, neg_m));
        psum += p0 + p1;
        __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&pk);
      }
      l_sum = l_sum * factor + psum;

      // P and O may be touched only after the previous P.V has finished
      if (j > 0) {
        got = 1;
        if (lane == 0) got = sm100::mbar_wait(&ctl.p_empty, (j - 1) & 1, abort_flag, p.status, kWaitPEmpty);
        if (!__shfl_sync(0xffffffffu, got, 0)) { ok = false; break; }
        sm100::tc_fence_after_sync();
      }
      // lanes 16-31 hold the upper 256 output columns of the row owned by lane - 16
      const float my_factor = __shfl_sync(0xffffffffu, factor, lane & 15);
      if (__any_sync(0xffffffffu, my_factor != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < 256; c += 32) {
          uint32_t o[32];
          sm100::tmem_ld_32x32(lane_base + kColO + c, o);
          sm100::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * my_factor);
          tmem_st_32x32(lane_base + kColO + c, o);
        }
        tmem_st_wait();
      }
      if (row_ok) {
        const int r = warp * 16 + lane;
        uint8_t* prow = p_tile + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) =
              make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      }
      sm100::fence_proxy_async();
      sm100::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&ctl.p_full);
    }

    // ------------------------------------------------------------ epilogue
    if (ok) {
      int got = 1;
      if (lane == 0) got = sm100::mbar_wait(&ctl.o_done, 0, abort_flag, p.status, kWaitODone);
      ok = __shfl_sync(0xffffffffu, got, 0) != 0;
    }
    if (ok) {
      sm100::tc_fence_after_sync();
      const float l_row = __shfl_sync(0xffffffffu, l_sum, lane & 15);
      const float m_row = __shfl_sync(0xffffffffu, m_ref, lane & 15);
      const int col0 = lane < 16 ? 0 : 256;
      if (p.nsplit == 1) {
        const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
        __nv_bfloat16* dst = p.out + ((size_t)b * p.Hh + head) * kDv + col0;
#pragma unroll 1
        for (int c = 0; c < 256; c += 32) {
          uint32_t o[32];
          if (nb > 0) { sm100::tmem_ld_32x32(lane_base + kColO + c, o); sm100::tmem_ld_wait(); }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float a = nb > 0 ? __uint_as_float(o[8 * v + 2 * k]) * inv : 0.f;
              const float bb = nb > 0 ? __uint_as_float(o[8 * v + 2 * k + 1]) * inv : 0.f;
              __nv_bfloat162 pk = __floats2bfloat162_rn(l_row > 0.f ? a : 0.f, l_row > 0.f ? bb : 0.f);
              w[k] = *reinterpret_cast<uint32_t*>(&pk);
            }
            *reinterpret_cast<uint4*>(dst + c + 8 * v) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      } else {
        const size_t slot = ((size_t)b * p.nsplit + split) * p.Hh + head;
        float* dst = p.part_o + slot * kDv + col0;
#pragma unroll 1
        for (int c = 0; c < 256; c += 32) {
          uint32_t o[32];
          if (nb > 0) { sm100::tmem_ld_32x32(lane_base + kColO + c, o); sm100::tmem_ld_wait(); }
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            float4 f;
            f.x = (nb > 0 && l_row > 0.f) ? __uint_as_float(o[4 * v + 0]) : 0.f;
            f.y = (nb > 0 && l_row > 0.f) ? __uint_as_float(o[4 * v + 1]) : 0.f;
            f.z = (nb > 0 && l_row > 0.f) ? __uint_as_float(o[4 * v + 2]) : 0.f;
            f.w = (nb > 0 && l_row > 0.f) ? __uint_as_float(o[4 * v + 3]) : 0.f;
            *reinterpret_cast<float4*>(dst + c + 4 * v) = f;
          }
        }
        if (lane < 16) {
          p.part_ml[slot * 2 + 0] = m_row;
          p.part_ml[slot * 2 + 1] = l_row;
        }
      }
    }
  }

  sm100::tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    sm100::tc_fence_after_sync();
    sm100::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair kernel: 128 query heads of one sequence on a cluster of two CTAs that split the 576
// columns of the cache rows between them.
//
//   CTA r holds value columns [256 r, 256 r + 256) and rotary columns [512 + 32 r, +32) of Q (128
//   heads) and of every gathered row, so each selected row crosses the L2 -> SM path once per
//   sequence and a stage of 64 rows takes 36 KB instead of 72 KB: four 64-column tiles in the
//   128-byte swizzle plus one 32-column tile in the 64-byte swizzle. The 256 value columns of Q live
//   in tensor memory (the A operand of tcgen05.mma may come from there: lane = head, two bf16 per
//   32-bit column); only its 32 rotary columns stay in shared memory. That leaves room for four
//   stages. A stage lands in two parts with a barrier each, so Q.K^T starts on the first part while
//   the rest of the block is still in flight.
//   S = Q . K^T is computed as two partial sums over those column ranges, M=128 N=64 (twice the
//   heads per instruction of the single-CTA kernel at the same cost). Four exchange warps read
//   their CTA's partial from tensor memory, store it into the other CTA's exchange buffer through
//   distributed shared memory, add what the other CTA stored here and write the complete scores
//   back to tensor memory, ahead of the softmax. Both CTAs hold the same fp32 scores (a sum of two
//   terms does not depend on their order) and run the same softmax.
//   O = P . V: each CTA accumulates 128 heads x its 256 of the 512 value columns (the first 256
//   columns of its slice), M=128 N=256.
//   Eight softmax warps in two groups that take the blocks in turn; warp w works on the 32 heads of
//   lane quadrant w % 4, one thread per head.
// Every wait is bounded; a CTA that gives up still reaches the closing cluster barrier, so its
// partner's stores never hit shared memory of a CTA that has exited.
constexpr int kPairHeads = 128;
constexpr int kPairThreads = 22 * 32;              // 8 softmax, Q.K^T issuer, 4 producer, 4 sending, P.V issuer, 4 receiving warps
constexpr int kPairStages = 4;
constexpr int kPairTiles = 2;                      // a stage lands in two parts: value tiles 0,1, then 2,3 and the rotary tile
constexpr int kPairQRopeBytes = kPairHeads * 64;   // 128 heads x 32 rotary columns
constexpr int kPairRopeOffset = 4 * kChunkBytes;   // rotary tile of a stage: 64 rows x 64 bytes
constexpr int kPairStageBytes = kPairRopeOffset + kTok * 64;   // 36864
constexpr int kPairXBytes = kPairHeads * kTok * 4; // partial scores of the other CTA
constexpr int kPairPBytes = kPairHeads * 128;      // P: 128 heads x 64 tokens bf16
constexpr uint32_t kPairColS = 0, kPairColQ = 128, kPairColO = 256;

struct __align__(16) PairControl {
  uint64_t kv_full[kPairStages][kPairTiles], kv_empty[kPairStages], s_full[2], s_copied[2][2], s_ready[2], s_empty[2], p_full[2], p_empty[2],
      x_full[2][2], x_free[2], o_done;   // p_full, p_empty, x_full: [even / odd blocks]; x_full, x_free: [.. column half]
  uint64_t pub[4][2];                // [lane quadrant][even / odd blocks]: the row references after that block are published
  uint64_t duo[4];                   // the two softmax warps of a lane quadrant meet here (64 arrivals)
  uint32_t tmem_base;
  int abort_flag;
  unsigned char valid[kPairStages][kTok];
  float row_ref[kPairHeads];         // reference maximum of each head (log2 units) as the last block left it
  float row_sum[2][kPairHeads];      // [softmax group][head], used once at the end
};
constexpr int kPairSmemBytes = kPairQRopeBytes + kPairStages * kPairStageBytes + kPairXBytes + 2 * kPairPBytes +
                               (int)sizeof(PairControl) + 1024;

enum { kWaitXFull = 208, kWaitXFree = 209, kWaitDuo = 210 };

// 2^x for x <= 0 (and -inf -> 0) in one special-function instruction; results below 2^-126 become 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Operand descriptor for K-major tiles with rows of 64 bytes in the 64-byte swizzle (16-byte unit u of row r
// sits at unit u ^ ((r >> 1) & 3)); groups of 8 rows are 512 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw64(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(512 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)4 << 61);
}

// D[tmem] (+)= A[tmem] * B[smem]^T: the A operand (128 lanes x 8 columns = 128 x 16 bf16) is read from
// tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Producer warp `pw` (0..3) of the pair kernel: rows [16 pw, +16) of every block. A warp needs about
// 100 clk per 16-byte-per-lane cp.async instruction whatever the number of warps copying, so the four
// warps share each block (18 instructions each) instead of taking blocks in turn (36 each).
// The block is copied as two cp.async groups (value tiles 0 and 1; value tiles 2, 3 and the rotary tile),
// each published on its own barrier as soon as it has landed.
__device__ __forceinline__ void pair_produce(const MlaParams& p, PairControl& ctl, uint8_t* kv_tile, int pw,
                                             int lane, int b, int j0, int nb, int len, int rank) {
  volatile int* abort_flag = &ctl.abort_flag;
  const int* idx_b = p.idx + (size_t)b * p.topk;
  const uint8_t* kv_b = reinterpret_cast<const uint8_t*>(p.kv + (size_t)(b / p.Sq) * p.S * kDqk);   // b: (sequence, query token)
  const int vbyte0 = rank * 512, rbyte0 = 1024 + rank * 64;
  // The cache row number of this lane's row (lanes l and l+16 hold the same one) is fetched one block
  // early, and the slices of rows further ahead are requested into L2 by lanes 0-15, so that the copies
  // into shared memory mostly hit L2.
  constexpr int kPrefetchAhead = 4;
  auto entry = [&](int j) {
    const int i = (j0 + j) * kTok + pw * 16 + (lane & 15);
    return (j < nb && i < p.topk) ? __ldg(idx_b + i) : -1;
  };
  auto prefetch = [&](int t) {
    if (lane < 16 && t >= 0 && t < len) {   // rows start on 128-byte lines: four lines of value columns, one with the rotary ones
      const uint8_t* row = kv_b + (size_t)t * (kDqk * 2);
#pragma unroll
      for (int l = 0; l < 4; ++l) sm100::prefetch_l2_line(row + vbyte0 + l * 128);
      sm100::prefetch_l2_line(row + rbyte0);
    }
  };
  for (int a = 1; a <= kPrefetchAhead; ++a) prefetch(entry(a));
  // every row number is loaded an iteration before it is used, so that no iteration waits for the load
  int t_next = entry(0), t_prefetch = entry(kPrefetchAhead + 1);
  for (int j = 0; j < nb; ++j) {
    const int st = j % kPairStages, use = j / kPairStages;
    const int my_t = t_next, pf_t = t_prefetch;
    t_next = entry(j + 1);
    t_prefetch = entry(j + kPrefetchAhead + 2);
    prefetch(pf_t);
    if (use >= 1 && !sm100::mbar_wait_relaxed(&ctl.kv_empty[st], (use - 1) & 1, abort_flag, p.status, kWaitKvEmpty))
      break;
    const uint32_t dst = sm100::smem_u32(kv_tile + st * kPairStageBytes);
    const bool my_ok = my_t >= 0 && my_t < len;
    if (lane < 16) ctl.valid[st][pw * 16 + lane] = my_ok ? 1 : 0;
    const int my_row = my_ok ? my_t : 0;   // an invalid entry copies row 0: finite data under a zero weight
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int piece = it * 32 + lane;
        const int rl = piece >> 3, c16 = piece & 7;
        const int r = pw * 16 + rl;
        const int t = __shfl_sync(0xffffffffu, my_row, rl);
        cp_async_16(dst + c * kChunkBytes + r * 128 + ((c16 ^ (r & 7)) << 4),
                    kv_b + (size_t)t * (kDqk * 2) + vbyte0 + c * 128 + c16 * 16);
      }
      if (c == 1) cp_async_commit();
    }
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int piece = it * 32 + lane;
      const int rl = piece >> 2, c16 = piece & 3;
      const int r = pw * 16 + rl;
      const int t = __shfl_sync(0xffffffffu, my_row, rl);
      cp_async_16(dst + kPairRopeOffset + r * 64 + ((c16 ^ ((r >> 1) & 3)) << 4),
                  kv_b + (size_t)t * (kDqk * 2) + rbyte0 + c16 * 16);
    }
    cp_async_commit();
    cp_async_wait<1>(); sm100::fence_proxy_async(); sm100::mbar_arrive(&ctl.kv_full[st][0]);
    cp_async_wait<0>(); sm100::fence_proxy_async(); sm100::mbar_arrive(&ctl.kv_full[st][1]);
  }
}

// The same with TMA row gathers (cp.async.bulk.tensor ... tile::gather4): one instruction fetches this CTA's
// 128-byte (or, for the rotary tile, 64-byte) piece of four selected rows straight into its place in the
// swizzled tile. Warp pw still owns rows [16 pw, +16) of every block: lanes 0..19 issue one gather each
// (tile = lane / 4: four value tiles and the rotary tile; four rows = 4 (lane % 4) .. +3), lane 0 posts the
// bytes the warp's gathers will deliver on the stage's two barriers. Nothing passes through registers and no
// thread waits for the data.
__device__ __forceinline__ void pair_produce_tma(const MlaParams& p, PairControl& ctl, uint8_t* kv_tile, int pw,
                                                 int lane, int b, int j0, int nb, int len, int rank,
                                                 const CUtensorMap* map_v, const CUtensorMap* map_r) {
  volatile int* abort_flag = &ctl.abort_flag;
  const int* idx_b = p.idx + (size_t)b * p.topk;
  const int seq = b / p.Sq;                                   // b: (sequence, query token)
  const int row_base = seq * p.S;                             // the cache as one [B * S, 576] tensor
  const uint8_t* kv_b = reinterpret_cast<const uint8_t*>(p.kv + (size_t)seq * p.S * kDqk);
  const int vbyte0 = rank * 512, rbyte0 = 1024 + rank * 64;
  constexpr int kPrefetchAhead = 4;
  auto entry = [&](int j) {
    const int i = (j0 + j) * kTok + pw * 16 + (lane & 15);
    return (j < nb && i < p.topk) ? __ldg(idx_b + i) : -1;
  };
  auto prefetch = [&](int t) {
    if (lane < 16 && t >= 0 && t < len) {
      const uint8_t* row = kv_b + (size_t)t * (kDqk * 2);
#pragma unroll
      for (int l = 0; l < 4; ++l) sm100::prefetch_l2_line(row + vbyte0 + l * 128);
      sm100::prefetch_l2_line(row + rbyte0);
    }
  };
  for (int a = 1; a <= kPrefetchAhead; ++a) prefetch(entry(a));
  int t_next = entry(0), t_prefetch = entry(kPrefetchAhead + 1);
  const int tile = lane >> 2, quad4 = lane & 3;
  for (int j = 0; j < nb; ++j) {
    const int st = j % kPairStages, use = j / kPairStages;
    const int my_t = t_next, pf_t = t_prefetch;
    t_next = entry(j + 1);
    t_prefetch = entry(j + kPrefetchAhead + 2);
    prefetch(pf_t);
    if (use >= 1 && !sm100::mbar_wait_relaxed(&ctl.kv_empty[st], (use - 1) & 1, abort_flag, p.status, kWaitKvEmpty))
      break;
    const bool my_ok = my_t >= 0 && my_t < len;
    if (lane < 16) ctl.valid[st][pw * 16 + lane] = my_ok ? 1 : 0;
    const int my_row = row_base + (my_ok ? my_t : 0);   // an invalid entry fetches row 0: finite data under a zero weight
    const int r0 = __shfl_sync(0xffffffffu, my_row, 4 * quad4 + 0), r1 = __shfl_sync(0xffffffffu, my_row, 4 * quad4 + 1);
    const int r2 = __shfl_sync(0xffffffffu, my_row, 4 * quad4 + 2), r3 = __shfl_sync(0xffffffffu, my_row, 4 * quad4 + 3);
    if (lane == 0) {
      sm100::mbar_arrive_expect_tx(&ctl.kv_full[st][0], 2 * 16 * 128);
      sm100::mbar_arrive_expect_tx(&ctl.kv_full[st][1], 2 * 16 * 128 + 16 * 64);
    }
    __syncwarp();
    uint8_t* dst = kv_tile + st * kPairStageBytes;
    const int first = pw * 16 + 4 * quad4;
    if (tile < 4)
      sm100::tma_gather4_2d(dst + tile * kChunkBytes + first * 128, map_v, &ctl.kv_full[st][tile >> 1],
                            rank * 256 + tile * 64, r0, r1, r2, r3);
    else if (tile == 4)
      sm100::tma_gather4_2d(dst + kPairRopeOffset + first * 64, map_r, &ctl.kv_full[st][1], 512 + rank * 32, r0, r1, r2,
                            r3);
  }
}

template <bool kTmaGather>
__global__ void __cluster_dims__(2, 1, 1) __maxnreg__(80)
mla_sparse_decode_pair_kernel(const MlaParams p, const __grid_constant__ CUtensorMap map_v,
                              const __grid_constant__ CUtensorMap map_r) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_rope = base;                              // this CTA's 32 rotary columns of Q, 128 heads x 64 bytes
  uint8_t* kv_tile = q_rope + kPairQRopeBytes;         // four stages
  uint8_t* x_tile = kv_tile + kPairStages * kPairStageBytes;   // float4 [16 column groups][128 heads]
  uint8_t* p_tile = x_tile + kPairXBytes;
  PairControl& ctl = *reinterpret_cast<PairControl*>(p_tile + 2 * kPairPBytes);   // two P tiles (even / odd blocks)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = sm100::cluster_ctarank(), peer = rank ^ 1u;
  const int head0 = (blockIdx.x >> 1) * kPairHeads, split = blockIdx.y, b = blockIdx.z;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      for (int c = 0; c < kPairTiles; ++c) sm100::mbar_init(&ctl.kv_full[s][c], kTmaGather ? 4 : 128);
      sm100::mbar_init(&ctl.kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      sm100::mbar_init(&ctl.s_full[s], 1);
      sm100::mbar_init(&ctl.s_copied[s][0], 4);       // the sending warps have read a half of the partial scores
      sm100::mbar_init(&ctl.s_copied[s][1], 4);
      sm100::mbar_init(&ctl.s_ready[s], 4);           // the receiving warps have completed the scores
      sm100::mbar_init(&ctl.s_empty[s], 4);           // the softmax warps of one group have read them
    }
    sm100::mbar_init(&ctl.p_full[0], 4);
    sm100::mbar_init(&ctl.p_full[1], 4);
    for (int s = 0; s < 8; ++s) sm100::mbar_init(&ctl.pub[s >> 1][s & 1], 1);
    sm100::mbar_init(&ctl.p_empty[0], 1);
    sm100::mbar_init(&ctl.p_empty[1], 1);
    for (int s = 0; s < 4; ++s) sm100::mbar_init(&ctl.x_full[s >> 1][s & 1], 1);   // one local arrival posts the bytes
    sm100::mbar_init(&ctl.x_free[1], 4);
    sm100::mbar_init(&ctl.x_free[0], 4);
    for (int s = 0; s < 4; ++s) sm100::mbar_init(&ctl.duo[s], 64);
    sm100::mbar_init(&ctl.o_done, 1);
    ctl.abort_flag = 0;
    sm100::mbar_fence_init();
    for (int s = 0; s < 4; ++s)   // partial scores of blocks 0 and 1 from the other CTA, in two column halves each
      sm100::mbar_arrive_expect_tx(&ctl.x_full[s >> 1][s & 1], kPairXBytes / 2);
  }
  if (threadIdx.x < kPairHeads) ctl.row_ref[threadIdx.x] = -INFINITY;
  if (warp == 8) {
    sm100::tmem_alloc(&ctl.tmem_base, kTmemCols);
    sm100::tmem_relinquish();
  }
  const uint8_t* q_rows = reinterpret_cast<const uint8_t*>(p.q + ((size_t)b * p.Hh + head0) * kDqk);
  if (threadIdx.x < kPairHeads * 4) {
    // this CTA's 32 rotary columns of Q as one tile in the 64-byte swizzle
    const int r = threadIdx.x >> 2, c16 = threadIdx.x & 3;
    cp_async_16(sm100::smem_u32(q_rope) + r * 64 + ((c16 ^ ((r >> 1) & 3)) << 4),
                q_rows + (size_t)r * (kDqk * 2) + 1024 + rank * 64 + c16 * 16);
    cp_async_commit();
    cp_async_wait<0>();
    sm100::fence_proxy_async();
  }
  sm100::tc_fence_before_sync();
  __syncthreads();
  sm100::tc_fence_after_sync();
  const uint32_t tmem_base = ctl.tmem_base;
  if (warp < 4) {
    // the 256 value columns of Q into tensor memory: thread = head = lane, 64 columns (128 bytes) per store
    const uint4* src = reinterpret_cast<const uint4*>(q_rows + (size_t)(warp * 32 + lane) * (kDqk * 2) + rank * 512);
    const uint32_t dst = tmem_base + ((uint32_t)(warp * 32) << 16) + kPairColQ;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t w[32];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint4 v = __ldg(src + c * 8 + u);
        w[4 * u] = v.x; w[4 * u + 1] = v.y; w[4 * u + 2] = v.z; w[4 * u + 3] = v.w;
      }
      tmem_st_32x32(dst + c * 32, w);
    }
    tmem_st_wait();
  }
  sm100::tc_fence_before_sync();
  __syncthreads();
  sm100::cluster_sync_all();          // both CTAs' barriers exist before anything arrives on them remotely
  sm100::tc_fence_after_sync();
  volatile int* abort_flag = &ctl.abort_flag;

  const int blocks_total = (p.topk + kTok - 1) / kTok;
  const int per_split = (blocks_total + p.nsplit - 1) / p.nsplit;
  const int j0 = split * per_split;
  const int nb = max(0, min(blocks_total, j0 + per_split) - j0);
  const int len = min(__ldg(p.seq_len + b), p.S);   // a length past the cache's extent never reaches a row outside it

  if (warp >= 13 && warp <= 16) {
    // ---------------------------------------------------------------- exchange, sending side (one warp per lane quadrant)
    // Reads this CTA's partial scores from tensor memory 16 columns at a time and stores them into the
    // other CTA's exchange buffer with asynchronous stores that count their bytes on that CTA's barrier.
    // The buffer is used in two halves (score columns 0-31 and 32-63) with their own barriers, so that
    // the other CTA may refill one half while the second is still being read. Sending and receiving are
    // separate warps: the 32 KB of a block keep the path between the SMs busy for about 1.5 k clk, and
    // the receiving side's waits and arithmetic run beside it instead of after it.
    sm100::reg_dec<48>();
    const int quad = warp & 3;        // a warp reaches the tensor-memory lanes of quadrant warp % 4 only
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t peer_x = sm100::cluster_map(sm100::smem_u32(x_tile), peer);
    const uint32_t peer_bar0 = sm100::cluster_map(sm100::smem_u32(&ctl.x_full[0][0]), peer);   // [sb][half]: + 16 sb + 8 half
    bool ok = true;
    for (int j = 0; j < nb && ok; ++j) {
      const int sb = j & 1;
      if (!sm100::mbar_wait(&ctl.s_full[sb], (j >> 1) & 1, abort_flag, p.status, kWaitSFull)) ok = false;
      if (!__all_sync(0xffffffffu, ok)) break;
      sm100::tc_fence_after_sync();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        // the other CTA's half buffer is free once its receiving warps have read block j-1 out of it
        if (j >= 1 && !sm100::mbar_wait_cluster(&ctl.x_free[half], (j - 1) & 1, abort_flag, p.status, kWaitXFree))
          ok = false;
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        const uint32_t bar = peer_bar0 + 16 * sb + 8 * half;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t t[16];
          tmem_ld_32x16(lane_base + kPairColS + sb * kTok + half * 32 + c * 16, t);
          sm100::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i)
            sm100::st_async_v4(peer_x + (uint32_t)(((half * 8 + c * 4 + i) * kPairHeads + row) * 16), bar, t[4 * i],
                               t[4 * i + 1], t[4 * i + 2], t[4 * i + 3]);
        }
        // this half of the partial scores is in flight: the receiving warp may write the sums over it
        sm100::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(&ctl.s_copied[sb][half]);
      }
    }
  } else if (warp >= 18) {
    // ---------------------------------------------------------------- exchange, receiving side (one warp per lane quadrant)
    // Adds what the other CTA stored here to this CTA's partial scores, 16 columns at a time, writes the
    // complete scores over the partial ones in tensor memory for the softmax warps and hands each half
    // of the buffer back as soon as it has been read.
    sm100::reg_dec<56>();
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t peer_free0 = sm100::cluster_map(sm100::smem_u32(&ctl.x_free[0]), peer);
    const float4* x_own = reinterpret_cast<const float4*>(x_tile);
    bool ok = true;
    for (int j = 0; j < nb && ok; ++j) {
      const int sb = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!sm100::mbar_wait(&ctl.s_full[sb], ph, abort_flag, p.status, kWaitSFull)) ok = false;
      if (!__all_sync(0xffffffffu, ok)) break;
      sm100::tc_fence_after_sync();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (!sm100::mbar_wait(&ctl.x_full[sb][half], ph, abort_flag, p.status, kWaitXFull) ||
            !sm100::mbar_wait(&ctl.s_copied[sb][half], ph, abort_flag, p.status, kWaitSFull))
          ok = false;
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        sm100::tc_fence_after_sync();
        if (quad == 0 && lane == 0 && j + 2 < nb)
          sm100::mbar_arrive_expect_tx(&ctl.x_full[sb][half], kPairXBytes / 2);   // block j+2
        {
          // both 16-column loads of the half are issued before the wait, so that their round trips overlap
          uint32_t t[32];
          uint32_t (&ta)[16] = *reinterpret_cast<uint32_t(*)[16]>(&t[0]);
          uint32_t (&tb)[16] = *reinterpret_cast<uint32_t(*)[16]>(&t[16]);
          tmem_ld_32x16(lane_base + kPairColS + sb * kTok + half * 32, ta);
          tmem_ld_32x16(lane_base + kPairColS + sb * kTok + half * 32 + 16, tb);
          sm100::tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            float4 xa[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xa[i] = x_own[(half * 8 + c * 4 + i) * kPairHeads + row];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t* d4 = &t[c * 16 + 4 * i];
              d4[0] = __float_as_uint(__uint_as_float(d4[0]) + xa[i].x);
              d4[1] = __float_as_uint(__uint_as_float(d4[1]) + xa[i].y);
              d4[2] = __float_as_uint(__uint_as_float(d4[2]) + xa[i].z);
              d4[3] = __float_as_uint(__uint_as_float(d4[3]) + xa[i].w);
            }
          }
          tmem_st_32x16(lane_base + kPairColS + sb * kTok + half * 32, ta);
          tmem_st_32x16(lane_base + kPairColS + sb * kTok + half * 32 + 16, tb);
        }
        // every value read from this half has been used: it may be overwritten
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive_cluster_relaxed(peer_free0 + 8 * half);
      }
      if (!ok) break;
      tmem_st_wait();
      sm100::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&ctl.s_ready[sb]);
    }
  } else if (warp >= 9 && warp <= 12) {
    // ---------------------------------------------------------------- producers
    // each warp owns 16 of every block's 64 rows and copies this CTA's slice of them (36 sixteen-byte
    // pieces per row)
    sm100::reg_dec<56>();
    if (kTmaGather)
      pair_produce_tma(p, ctl, kv_tile, warp - 9, lane, b, j0, nb, len, (int)rank, &map_v, &map_r);
    else
      pair_produce(p, ctl, kv_tile, warp - 9, lane, b, j0, nb, len, (int)rank);
  } else if (warp == 8) {
    // ---------------------------------------------------------------- Q.K^T issuer
    // Two issuing threads (this one and the P.V issuer in warp 17) instead of one that polls: each
    // simply waits for what it needs next, and the tensor core takes their instructions as they come.
    sm100::reg_dec<40>();
    if (lane == 0) {
      constexpr uint32_t idesc_qk = sm100::umma_idesc(1 /* bf16 */, kPairHeads, kTok);
      const uint64_t a_rope = umma_desc_sw64(sm100::smem_u32(q_rope));
      for (int j = 0; j < nb; ++j) {
        const int st = j % kPairStages, sb = j & 1;
        const uint32_t ph = (j / kPairStages) & 1;
        const uint32_t k_addr = sm100::smem_u32(kv_tile + st * kPairStageBytes);
        const uint32_t d = tmem_base + kPairColS + sb * kTok;
        if (!sm100::mbar_wait(&ctl.s_empty[sb], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kWaitSEmpty)) break;
        bool ok = true;
#pragma unroll
        for (int c = 0; c < 4 && ok; ++c) {
          if ((c & 1) == 0) {
            if (!sm100::mbar_wait(&ctl.kv_full[st][c >> 1], ph, abort_flag, p.status, kWaitKvFull)) { ok = false; break; }
            sm100::tc_fence_after_sync();
          }
          const uint64_t bd = umma_desc_sw128(k_addr + c * kChunkBytes, 16, 1024);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_f16_ts(d, tmem_base + kPairColQ + c * 32 + k4 * 8, bd + 2 * k4, idesc_qk, (c > 0 || k4 > 0) ? 1u : 0u);
        }
        if (!ok) break;
        const uint64_t bd = umma_desc_sw64(k_addr + kPairRopeOffset);
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2) sm100::umma_f16(d, a_rope + 2 * k2, bd + 2 * k2, idesc_qk, 1u);
        sm100::umma_commit(&ctl.s_full[sb]);
      }
    }
    __syncwarp();
  } else if (warp == 17) {
    // ---------------------------------------------------------------- P.V issuer
    sm100::reg_dec<40>();
    if (lane == 0) {
      constexpr uint32_t idesc_pv = sm100::umma_idesc(1, kPairHeads, 256) | (1u << 16);   // B is MN-major
      bool ok = true;
      for (int j = 0; j < nb; ++j) {
        const int st = j % kPairStages;
        if (!sm100::mbar_wait(&ctl.p_full[j & 1], (j >> 1) & 1, abort_flag, p.status, kWaitPFull)) { ok = false; break; }
        const uint64_t a = umma_desc_sw128(sm100::smem_u32(p_tile + (j & 1) * kPairPBytes), 16, 1024);
        sm100::tc_fence_after_sync();
        const uint64_t bd = umma_desc_sw128(sm100::smem_u32(kv_tile + st * kPairStageBytes), kChunkBytes, 1024);
#pragma unroll
        for (int k4 = 0; k4 < kTok / 16; ++k4)
          sm100::umma_f16(tmem_base + kPairColO, a + 2 * k4, bd + (uint64_t)k4 * (2048 >> 4), idesc_pv,
                          (j > 0 || k4 > 0) ? 1u : 0u);
        sm100::umma_commit(&ctl.kv_empty[st]);      // the stage may be refilled
        sm100::umma_commit(&ctl.p_empty[j & 1]);    // P and O may be touched again
      }
      if (ok) sm100::umma_commit(&ctl.o_done);
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax + epilogue (warps 0..7)
    // 22 warps launch with 80 registers per thread. Registers are handed over inside each SM
    // sub-partition (warps w, w+4, w+8, ...: two softmax warps, a producer, a sending and a receiving
    // warp, and an issuing warp in sub-partitions 0 and 1): 2 x 120 + 56 + 48 + 56 (+ 40) <= 5 (6) x 80.
    sm100::reg_inc<120>();
    // Two groups of four warps take the blocks in turn (group 0 the even ones, group 1 the odd ones), one
    // thread per head with all 64 scores of the block, so that the waits of one block hide behind the
    // arithmetic of the other. Each group has its own P tile. What orders the blocks is a small barrier per
    // lane quadrant: a warp finishes block j only after the other group's warp of the same quadrant has
    // published the rows' reference maxima after block j-1; then the thread reads its row's reference,
    // decides about raising it, and publishes it for block j+1. The exponentials are computed earlier
    // against the reference the thread could see then, and once more in the rare case that it changed.
    const int quad = warp & 3, grp = warp >> 2;
    const int row = quad * 32 + lane;                  // head inside the 128; tensor-memory lane
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    volatile float* m_shared = ctl.row_ref;
    float m_loc = -INFINITY, l_part = 0.f;             // this thread's sum is relative to m_loc
    bool ok = true;
    for (int j = grp; j < nb; j += 2) {
      const int sb = j & 1, st = j % kPairStages;
      if (!sm100::mbar_wait(&ctl.s_ready[sb], (j >> 1) & 1, abort_flag, p.status, kWaitSFull)) { ok = false; }
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      sm100::tc_fence_after_sync();
      uint32_t t[64];
      {
        uint32_t (&t0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&t[0]);
        uint32_t (&t1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&t[32]);
        sm100::tmem_ld_32x32(lane_base + kPairColS + sb * kTok, t0);
        sm100::tmem_ld_32x32(lane_base + kPairColS + sb * kTok + 32, t1);
      }
      sm100::tmem_ld_wait();
      sm100::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&ctl.s_empty[sb]);

      const unsigned v_lo = __ballot_sync(0xffffffffu, ctl.valid[st][lane] != 0);
      const unsigned v_hi = __ballot_sync(0xffffffffu, ctl.valid[st][32 + lane] != 0);
      if ((v_lo & v_hi) != 0xffffffffu) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (!(((i < 32 ? v_lo : v_hi) >> (i & 31)) & 1u)) t[i] = __float_as_uint(-INFINITY);
      }
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 64; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(t[i]));
      const float m_blk = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;   // scale > 0

      // reference after this block, given the reference before it: raised on the first non-empty block
      // or on a jump of more than 2^8
      auto next_ref = [&](float before) {
        if (m_blk == -INFINITY) return before;
        if (before == -INFINITY || m_blk > before + kRescaleThreshold) return m_blk;
        return before;
      };
      uint32_t packed[32];
      float psum;
      auto exponentials = [&](float ref) {
        const float neg_m = ref == -INFINITY ? 0.f : -ref;   // exp2(-inf) = 0 for masked entries
        float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(t[i]), p.scale_log2, neg_m));
          const float p1 = fast_exp2(fmaf(__uint_as_float(t[i + 1]), p.scale_log2, neg_m));
          ps4[(i >> 1) & 3] += p0 + p1;
          __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&pk);
        }
        psum = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      };
      const float m_guess = next_ref(m_shared[row]);   // block j-1 may not have published yet
      exponentials(m_guess);

      // This block's P tile (one for the even, one for the odd blocks) is free once P.V of block j-2 has
      // finished; the row references are final once block j-1 has published them.
      if (j >= 2 && !sm100::mbar_wait(&ctl.p_empty[j & 1], ((j - 2) >> 1) & 1, abort_flag, p.status, kWaitPEmpty))
        ok = false;
      if (j >= 1 && !sm100::mbar_wait(&ctl.pub[quad][(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, p.status, kWaitDuo))
        ok = false;
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      const float m_prev = m_shared[row];
      const float m_new = next_ref(m_prev);
      if (m_new != m_guess) exponentials(m_new);
      // O holds sums relative to m_prev
      const float factor = (m_prev != -INFINITY && m_new != m_prev) ? exp2f(m_prev - m_new) : 1.f;
      if (__any_sync(0xffffffffu, factor != 1.f)) {
        // rare: O is rescaled in place, which needs P.V of block j-1 to have finished
        if (j >= 1 && !sm100::mbar_wait(&ctl.p_empty[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, p.status, kWaitPEmpty))
          ok = false;
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        sm100::tc_fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < 256; c += 32) {
          uint32_t o[32];
          sm100::tmem_ld_32x32(lane_base + kPairColO + c, o);
          sm100::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          tmem_st_32x32(lane_base + kPairColO + c, o);
        }
        tmem_st_wait();
      }
      if (m_loc != m_new) {
        l_part = m_loc == -INFINITY ? 0.f : l_part * exp2f(m_loc - m_new);
        m_loc = m_new;
      }
      l_part += psum;
      m_shared[row] = m_new;
      {
        uint8_t* prow = p_tile + (j & 1) * kPairPBytes + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) =
              make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      }
      sm100::fence_proxy_async();
      sm100::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        sm100::mbar_arrive(&ctl.pub[quad][j & 1]);      // the references of this warp's rows are final for block j
        sm100::mbar_arrive(&ctl.p_full[j & 1]);
      }
    }

    // ------------------------------------------------------------ epilogue
    if (ok && !sm100::mbar_wait(&ctl.o_done, 0, abort_flag, p.status, kWaitODone)) ok = false;
    ok = __all_sync(0xffffffffu, ok);
    // both groups are done: bring the two partial row sums to the final reference and add them
    float l_row = 0.f, m_fin = -INFINITY;
    if (ok) {
      sm100::mbar_arrive(&ctl.duo[quad]);
      if (!sm100::mbar_wait(&ctl.duo[quad], 0, abort_flag, p.status, kWaitDuo)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      m_fin = m_shared[row];
      ctl.row_sum[grp][row] = (m_loc == -INFINITY) ? 0.f : l_part * exp2f(m_loc - m_fin);
      sm100::mbar_arrive(&ctl.duo[quad]);
      if (!sm100::mbar_wait(&ctl.duo[quad], 1, abort_flag, p.status, kWaitDuo)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      l_row = ctl.row_sum[0][row] + ctl.row_sum[1][row];
    }
    if (ok) {
      sm100::tc_fence_after_sync();
      const int head = head0 + row;
      const int half = grp;                                // the two warps of a quadrant share the 256 columns
      const int col0 = (int)rank * 256 + half * 128;
      const bool live = nb > 0 && l_row > 0.f;
      if (p.nsplit == 1) {
        const float inv = live ? 1.f / l_row : 0.f;
        __nv_bfloat16* dst = p.out + ((size_t)b * p.Hh + head) * kDv + col0;
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
          uint32_t o[32];
          if (nb > 0) { sm100::tmem_ld_32x32(lane_base + kPairColO + half * 128 + c, o); sm100::tmem_ld_wait(); }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float a = live ? __uint_as_float(o[8 * v + 2 * k]) * inv : 0.f;
              const float bb = live ? __uint_as_float(o[8 * v + 2 * k + 1]) * inv : 0.f;
              __nv_bfloat162 pk = __floats2bfloat162_rn(a, bb);
              w[k] = *reinterpret_cast<uint32_t*>(&pk);
            }
            *reinterpret_cast<uint4*>(dst + c + 8 * v) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      } else {
        const size_t slot = ((size_t)b * p.nsplit + split) * p.Hh + head;
        float* dst = p.part_o + slot * kDv + col0;
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
          uint32_t o[32];
          if (nb > 0) { sm100::tmem_ld_32x32(lane_base + kPairColO + half * 128 + c, o); sm100::tmem_ld_wait(); }
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            float4 f;
            f.x = live ? __uint_as_float(o[4 * v + 0]) : 0.f;
            f.y = live ? __uint_as_float(o[4 * v + 1]) : 0.f;
            f.z = live ? __uint_as_float(o[4 * v + 2]) : 0.f;
            f.w = live ? __uint_as_float(o[4 * v + 3]) : 0.f;
            *reinterpret_cast<float4*>(dst + c + 4 * v) = f;
          }
        }
        if (rank == 0 && half == 0) {
          p.part_ml[slot * 2 + 0] = m_fin;
          p.part_ml[slot * 2 + 1] = l_row;
        }
      }
    }
  }

  sm100::tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    sm100::tc_fence_after_sync();
    sm100::tmem_dealloc(tmem_base, kTmemCols);
  }
  sm100::cluster_sync_all();          // nobody leaves while the partner may still store into this CTA
}

// Merge of the per-split partials: out = sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s.
__global__ void __launch_bounds__(128)
mla_combine_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o,
                   const float* __restrict__ part_ml, int Hh, int nsplit) {
  const int bh = blockIdx.x;                // b * Hh + h
  const int b = bh / Hh, h = bh - b * Hh;
  float m = -INFINITY;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[(((size_t)b * nsplit + s) * Hh + h) * 2]);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const size_t slot = ((size_t)b * nsplit + s) * Hh + h;
    const float ms = part_ml[slot * 2], ls = part_ml[slot * 2 + 1];
    if (ls <= 0.f || ms == -INFINITY) continue;
    const float w = exp2f(ms - m);
    const float4 o = *reinterpret_cast<const float4*>(part_o + slot * kDv + threadIdx.x * 4);
    acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
    l += w * ls;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
  uint2 w2;
  w2.x = *reinterpret_cast<uint32_t*>(&lo);
  w2.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(out + (size_t)bh * kDv + threadIdx.x * 4) = w2;
}

// Index validation + row gather on its own: rows[b, j, :] = kv[b, idx[b, j], :] or zeros.
__global__ void __launch_bounds__(256)
mla_gather_rows_kernel(uint4* __restrict__ rows, const uint4* __restrict__ kv, const int* __restrict__ seq_len,
                       const int* __restrict__ idx, int S, int topk, long long total) {
  const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // one 16-byte piece each
  if (id >= total) return;
  const int piece = (int)(id % 72);
  const long long rowid = id / 72;
  const int b = (int)(rowid / topk);
  const int t = __ldg(idx + rowid);
  const bool ok = t >= 0 && t < min(__ldg(seq_len + b), S);
  rows[id] = ok ? __ldg(kv + ((size_t)b * S + t) * 72 + piece) : make_uint4(0, 0, 0, 0);
}

}  // namespace

extern "C" size_t mla_sparse_decode_scratch_bytes(int B, int Hh, int nsplit) {
  if (nsplit <= 1) return 0;
  return (size_t)B * nsplit * Hh * (kDv + 2) * sizeof(float);
}

extern "C" int mla_sparse_decode_multi_launcher(cab_bf16* out, const cab_bf16* q, const cab_bf16* kv,
                                                const int* seq_len, const int* idx, int B, int Sq, int Hh, int S,
                                                int topk, float softmax_scale, int nsplit, void* scratch, int* status,
                                                int config, cudaStream_t stream) {
  if (B == 0 || Sq == 0) return CAB_OK;
  if (B < 0 || Sq < 0) return CAB_ERR_BAD_ARGUMENT;
  if ((long long)B * Sq > 65535) return CAB_ERR_TOO_LARGE;
  B *= Sq;          // from here on B counts (sequence, query token) pairs; only the cache is indexed per sequence
  if (!out || !q || !kv || !seq_len || !idx) return CAB_ERR_BAD_ARGUMENT;
  if (B < 0 || Hh <= 0 || Hh % kHeads != 0 || S <= 0 || topk <= 0 || nsplit <= 0) return CAB_ERR_BAD_ARGUMENT;
  if (nsplit > 1 && !scratch) return CAB_ERR_BAD_ARGUMENT;
  if (B > 65535 || nsplit > 65535) return CAB_ERR_TOO_LARGE;
  if (!cab::aligned_to(out, 16) || !cab::aligned_to(q, 16) || !cab::aligned_to(kv, 16) ||
      (scratch && !cab::aligned_to(scratch, 16)))
    return CAB_ERR_MISALIGNED;
  MlaParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.kv = reinterpret_cast<const __nv_bfloat16*>(kv);
  p.seq_len = seq_len; p.idx = idx;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.part_o = static_cast<float*>(scratch);
  p.part_ml = p.part_o ? p.part_o + (size_t)B * nsplit * Hh * kDv : nullptr;
  p.Hh = Hh; p.S = S; p.topk = topk; p.nsplit = nsplit; p.Sq = Sq;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  if (status && cudaMemsetAsync(status, 0, sizeof(int), stream) != cudaSuccess) return CAB_ERR_LAUNCH;
  // config 1 forces the single-CTA kernel (64 heads per CTA); otherwise 128-head groups run on CTA pairs,
  // gathering rows with TMA (config 2: with 16-byte cp.async copies instead)
  if (config != 1 && Hh % kPairHeads == 0) {
    const dim3 grid(2 * (Hh / kPairHeads), nsplit, B);
    CUtensorMap map_v, map_r;
    const unsigned long long cache_rows = (unsigned long long)(B / Sq) * (unsigned long long)S;
    const bool tma = config != 2 && cache_rows <= 0x7fffffffULL &&
                     sm100::make_tmap_2d(&map_v, kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, cache_rows, kDqk, 1, 64,
                                         CU_TENSOR_MAP_SWIZZLE_128B) &&
                     sm100::make_tmap_2d(&map_r, kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, cache_rows, kDqk, 1, 32,
                                         CU_TENSOR_MAP_SWIZZLE_64B);
    if (tma) {
      if (!cab::ensure_dynamic_smem<&mla_sparse_decode_pair_kernel<true>>(kPairSmemBytes)) return CAB_ERR_LAUNCH;
      mla_sparse_decode_pair_kernel<true><<<grid, kPairThreads, kPairSmemBytes, stream>>>(p, map_v, map_r);
    } else {
      memset(&map_v, 0, sizeof(map_v));
      memset(&map_r, 0, sizeof(map_r));
      if (!cab::ensure_dynamic_smem<&mla_sparse_decode_pair_kernel<false>>(kPairSmemBytes)) return CAB_ERR_LAUNCH;
      mla_sparse_decode_pair_kernel<false><<<grid, kPairThreads, kPairSmemBytes, stream>>>(p, map_v, map_r);
    }
  } else {
    if (!cab::ensure_dynamic_smem<&mla_sparse_decode_kernel>(kSmemBytes)) return CAB_ERR_LAUNCH;
    mla_sparse_decode_kernel<<<dim3(Hh / kHeads, nsplit, B), kThreads, kSmemBytes, stream>>>(p);
  }
  int rc = cab::launch_status();
  if (rc != CAB_OK || nsplit == 1) return rc;
  mla_combine_kernel<<<B * Hh, 128, 0, stream>>>(p.out, p.part_o, p.part_ml, Hh, nsplit);
  return cab::launch_status();
}

extern "C" int mla_sparse_decode_launcher(cab_bf16* out, const cab_bf16* q, const cab_bf16* kv,
                                          const int* seq_len, const int* idx, int B, int Hh, int S, int topk,
                                          float softmax_scale, int nsplit, void* scratch, int* status, int config,
                                          cudaStream_t stream) {
  return mla_sparse_decode_multi_launcher(out, q, kv, seq_len, idx, B, 1, Hh, S, topk, softmax_scale, nsplit, scratch,
                                          status, config, stream);
}

extern "C" int mla_gather_rows_launcher(cab_bf16* rows, const cab_bf16* kv, const int* seq_len, const int* idx,
                                        int B, int S, int topk, int config, cudaStream_t stream) {
  (void)config;
  if (B == 0 || topk == 0) return CAB_OK;
  if (!rows || !kv || !seq_len || !idx || B < 0 || S <= 0 || topk < 0) return CAB_ERR_BAD_ARGUMENT;
  if (!cab::aligned_to(rows, 16) || !cab::aligned_to(kv, 16)) return CAB_ERR_MISALIGNED;
  const long long total = (long long)B * topk * 72;
  const long long blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return CAB_ERR_TOO_LARGE;
  mla_gather_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<uint4*>(rows),
                                                               reinterpret_cast<const uint4*>(kv), seq_len, idx, S,
                                                               topk, total);
  return cab::launch_status();
}

namespace {
// ------------------------------------------------------------------------------------------------
// Split decode without any allocation.
//
// Some hosts of this library cannot give the split-KV path its scratch buffer: a serving process
// that handed all device memory to its own arena at start-up and forbids cudaMalloc on the request
// path (an allocation may fail there, and it synchronises the device), or a plugin interface whose
// operator signature carries inputs and outputs only, with no workspace argument and no allocator
// to call. For them the partial results live in a fixed array inside this library's device image.
//
// The array costs kStaticScratchBytes of device memory on every GPU that loads the library, from
// load until the process exits, whether or not this entry point is ever called. It is shared by all
// calls on that GPU: two calls whose kernels can overlap on the device (different streams, or
// different host threads) race on it and must be serialised by the caller. It keeps whatever the
// last call left in it; nothing has to be cleared, because every slot the merge kernel reads was
// written by the decode kernel of the same call.
constexpr size_t kStaticScratchBytes = CAB_MLA_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_mla_static_scratch[kStaticScratchBytes];

// In host code `g_mla_static_scratch` is only a handle for the runtime, not a device address; the
// address has to be asked for, once per device, with that device current.
constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

int static_scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return CAB_ERR_LAUNCH;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_mla_static_scratch) != cudaSuccess || !addr) return CAB_ERR_LAUNCH;
    g_scratch_addr[dev] = addr;
  }
  *out = g_scratch_addr[dev];
  return CAB_OK;
}

}  // namespace

extern "C" int mla_sparse_decode_noalloc_launcher(cab_bf16* out, const cab_bf16* q, const cab_bf16* kv,
                                                  const int* seq_len, const int* idx, int B, int Hh, int S,
                                                  int topk, float softmax_scale, int nsplit, int* status,
                                                  int config, cudaStream_t stream) {
  if (B == 0) return CAB_OK;
  if (B < 0 || Hh <= 0 || nsplit <= 0) return CAB_ERR_BAD_ARGUMENT;
  // every factor is bounded before the product is formed, so it cannot wrap
  if (B > 65535 || nsplit > 65535 || Hh > 65535) return CAB_ERR_TOO_LARGE;
  // (B * nsplit * Hh) slots of 512 + 2 floats must fit the fixed array
  const unsigned long long need = (unsigned long long)B * (unsigned long long)nsplit * (unsigned long long)Hh *
                                  (kDv + 2) * sizeof(float);
  if (nsplit > 1 && need > kStaticScratchBytes) return CAB_ERR_TOO_LARGE;
  void* scratch = nullptr;
  if (nsplit > 1) {
    const int rc = static_scratch_address(&scratch);   // first call on a device looks the address up
    if (rc != CAB_OK) return rc;
  }
  return mla_sparse_decode_launcher(out, q, kv, seq_len, idx, B, Hh, S, topk, softmax_scale, nsplit, scratch,
                                    status, config, stream);
}
