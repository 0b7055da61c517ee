// Grouped FP8 (e4m3) GEMM with 1x128 / 128x128 fp32 block scales on the sm_100a
// tensor cores (tcgen05.mma, accumulators in tensor memory, operands staged by TMA).
//
//   mode 0 (gate/up):  for every 128-row tile of expert e and every 128-column block j
//                      of the intermediate size I:
//                        G = A . W13[e, 128j .. 128j+127, :]^T      (gate rows)
//                        U = A . W13[e, I+128j .. I+128j+127, :]^T  (up rows)
//                        h = silu(G) * U, re-quantised to e4m3 with one scale per row
//                        per 128 columns (the activation rule), written as the A
//                        operand of mode 1.
//   mode 1 (down):     Y = Hq . W2[e]^T, written as bf16, 256 columns per tile.
//
// Both are C[m, n] = sum_kb sa[m, kb] * sb[n/128, kb] * (Aq[m, kb-block] . Bq[n, kb-block]),
// kb running over 128-wide K blocks. The scales are arbitrary fp32 numbers (not the
// power-of-two block scales the hardware applies), so each K block's 128x256 partial
// product is produced on its own in tensor memory (4 x tcgen05.mma m128 n256 k32), read
// back by the epilogue warps and added into fp32 registers with its scale, while the
// tensor core already works on the next K block in the other half of tensor memory.
//
// CTA layout (384 threads, one persistent CTA per SM):
//   warp 0       TMA producer: A tile (128 rows x 128 B) and two B tiles per stage, 4 stages
//   warp 1       issues tcgen05.mma, releases smem stages / publishes accumulators by commit
//   warp 2       allocates and frees the 512 tensor-memory columns (2 accumulator stages)
//   warps 4..11  promotion + epilogue: thread = one accumulator row (its TMEM lane) and
//                128 of the tile's 256 columns
// Rows come from a padded row space in which every 128-row tile belongs to one expert
// (tile_expert[]); rows of a tile past the expert's population hold unspecified data, are
// computed like any other row and are never read back.
#include "cab_common.cuh"
#include "sm100_primitives.cuh"

#include <cuda_fp8.h>

namespace {

constexpr int kBM = 128, kBN = 256, kBK = 128;
// Pipeline depth and the size of the output staging tile (written by the epilogue warps in the
// TMA 128-byte-swizzle layout, then stored with TMA): mode 0 stages 128x128 e4m3, mode 1 128x256 bf16.
template <int MODE> struct ModeCfg;
template <> struct ModeCfg<0> { static constexpr int kStages = 4; static constexpr int kOutBytes = 128 * 128; };
template <> struct ModeCfg<1> { static constexpr int kStages = 3; static constexpr int kOutBytes = 128 * 256 * 2; };
constexpr int kMaxStages = 4;
constexpr int kATileBytes = kBM * kBK;              // 16 KiB
constexpr int kBHalfBytes = 128 * kBK;              // 16 KiB: one 128-row weight box
constexpr int kStageBytes = kATileBytes + 2 * kBHalfBytes;
constexpr int kThreads = 384;
constexpr int kEpilogueThreads = 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccCols = 256;

constexpr int kScaleSlots = 8;   // > pipeline stages + accumulator stages + 1, see the producer

struct __align__(16) Control {
  float sa_ring[kScaleSlots][kBM];   // activation scales of the K blocks in flight, one row block each
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t epi_bar[2];       // two rendezvous points of the 256 epilogue threads per tile
  uint32_t tmem_base;
  int abort_flag;
  float amax[2][2][kBM];
};
template <int MODE>
constexpr int smem_bytes() {
  return ModeCfg<MODE>::kStages * kStageBytes + ModeCfg<MODE>::kOutBytes + (int)sizeof(Control) + 1024;
}

struct GemmParams {
  const float* a_scales_t;   // [K/128][ld_rows]
  const float* b_scales;     // [E][Nw/128][K/128]
  const int* tile_expert;    // [max tiles] or null (dense: expert 0 everywhere)
  const int* num_tiles;      // device scalar or null
  int fixed_tiles;           // used when num_tiles is null
  int KB;                    // K / 128
  int NBw;                   // weight rows per expert / 128
  int Nw;                    // weight rows per expert
  int n_tiles;               // tiles per 128-row block along N
  int ld_rows;               // row pitch of both transposed scale tables
  int out_ld;                // row length of the output
  void* out;
  float* out_scales_t;       // mode 0 only: [out_ld/128][ld_rows]
  int* status;
};

// where-codes written to GemmParams::status when a bounded wait gives up
enum { kWaitEmpty = 101, kWaitFull = 102, kWaitTmemEmpty = 103, kWaitTmemFull = 104, kWaitEpilogue = 105 };

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
__device__ __forceinline__ uint32_t pack2_bf16(float a, float b) {
  __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&p);
}

// First TMEM column of chunk ch (32 columns) of an epilogue thread in column group g:
// mode 0 reads gate columns 64g..64g+63 then up columns 128+64g..; mode 1 reads 128g..128g+127.
template <int MODE>
__device__ __forceinline__ constexpr int chunk_col(int ch, int g) {
  return MODE == 0 ? (ch < 2 ? 64 * g + 32 * ch : 128 + 64 * g + 32 * (ch - 2)) : 128 * g + 32 * ch;
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
moe_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_out, const GemmParams p) {
  constexpr int kStages = ModeCfg<MODE>::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = tiles + kStages * kStageBytes;
  Control& ctl = *reinterpret_cast<Control*>(out_stage + ModeCfg<MODE>::kOutBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { sm100::mbar_init(&ctl.full[s], 1); sm100::mbar_init(&ctl.empty[s], 1); }
    for (int a = 0; a < 2; ++a) {
      sm100::mbar_init(&ctl.tmem_full[a], 1);
      sm100::mbar_init(&ctl.tmem_empty[a], kEpilogueThreads / 32);
      sm100::mbar_init(&ctl.epi_bar[a], kEpilogueThreads);
    }
    ctl.abort_flag = 0;
    sm100::mbar_fence_init();
    sm100::prefetch_tensormap(&tmap_a);
    sm100::prefetch_tensormap(&tmap_b);
    sm100::prefetch_tensormap(&tmap_out);
  }
  if (warp == 2) {
    sm100::tmem_alloc(&ctl.tmem_base, kTmemCols);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before_sync();
  __syncthreads();
  sm100::tc_fence_after_sync();
  const uint32_t tmem_base = ctl.tmem_base;
  volatile int* abort_flag = &ctl.abort_flag;

  const int num_m_tiles = p.num_tiles ? __ldg(p.num_tiles) : p.fixed_tiles;
  const int total_tiles = num_m_tiles * p.n_tiles;
  const int half_n = p.Nw >> 1;   // mode 0: I (gate rows first, up rows second)

  if (warp < 4) {
    sm100::reg_dec<56>();
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------ TMA producer
      // Besides the operand tiles, each stage brings the 128 activation scales of its K block into
      // sa_ring[it % 8]. The producer is at most kStages K blocks ahead of the MMA issuer, which is at
      // most 2 ahead of the epilogue, so a slot is rewritten only after the epilogue has read it.
      int stage = 0; uint32_t phase = 0;
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        const int m_tile = tile / p.n_tiles, n_tile = tile - m_tile * p.n_tiles;
        const int e = p.tile_expert ? __ldg(p.tile_expert + m_tile) : 0;
        const int brow0 = e * p.Nw + (MODE == 0 ? n_tile * 128 : n_tile * 256);
        const int brow1 = MODE == 0 ? brow0 + half_n : brow0 + 128;
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!sm100::mbar_wait(&ctl.empty[stage], phase ^ 1, abort_flag, p.status, kWaitEmpty)) break;
          uint8_t* dst = tiles + stage * kStageBytes;
          sm100::mbar_arrive_expect_tx(&ctl.full[stage], kStageBytes + kBM * 4);
          sm100::bulk_load_1d(ctl.sa_ring[it & (kScaleSlots - 1)],
                              p.a_scales_t + (size_t)kb * p.ld_rows + m_tile * kBM, kBM * 4, &ctl.full[stage]);
          sm100::tma_load_2d(dst, &tmap_a, &ctl.full[stage], kb * kBK, m_tile * kBM);
          sm100::tma_load_2d(dst + kATileBytes, &tmap_b, &ctl.full[stage], kb * kBK, brow0);
          sm100::tma_load_2d(dst + kATileBytes + kBHalfBytes, &tmap_b, &ctl.full[stage], kb * kBK, brow1);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
          ++it;
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc = sm100::umma_idesc(0 /* e4m3 */, kBM, kBN);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!sm100::mbar_wait(&ctl.tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, kWaitTmemEmpty)) break;
          if (!sm100::mbar_wait(&ctl.full[stage], phase, abort_flag, p.status, kWaitFull)) break;
          sm100::tc_fence_after_sync();
          const uint32_t a_addr = sm100::smem_u32(tiles + stage * kStageBytes);
          const uint64_t a_desc = sm100::umma_desc_k_sw128(a_addr);
          const uint64_t b_desc = sm100::umma_desc_k_sw128(a_addr + kATileBytes);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 32; ++k4)   // 32 bytes of K per instruction: +2 in 16-byte units
            sm100::umma_f8f6f4(tmem_base + acc * kAccCols, a_desc + 2 * k4, b_desc + 2 * k4, idesc, k4 > 0);
          sm100::umma_commit(&ctl.empty[stage]);
          sm100::umma_commit(&ctl.tmem_full[acc]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
          acc ^= 1; if (acc == 0) acc_phase ^= 1;
        }
      }
    }
  } else {
    // -------------------------------------------------------------- promotion + epilogue
    sm100::reg_inc<224>();
    const int ew = warp - 4;
    const int quad = ew & 3;          // TMEM lane quadrant this warp may read (== warp id % 4)
    const int g = ew >> 2;            // which 128 of the 256 tile columns
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    int acc = 0; uint32_t acc_phase = 0;
    int tile_iter = 0;
    uint32_t it = 0;   // K blocks consumed so far: indexes the activation-scale ring
    for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tile_iter) {
      const int m_tile = tile / p.n_tiles, n_tile = tile - m_tile * p.n_tiles;
      const int e = p.tile_expert ? __ldg(p.tile_expert + m_tile) : 0;
      const int grow = m_tile * kBM + row;
      // Weight scales of this thread's two 64-column segments, for every K block of the tile: lane l
      // keeps blocks l and l+32 and hands them out by shuffle (KB <= 64).
      const int nb0 = MODE == 0 ? n_tile : 2 * n_tile + g;
      const int nb1 = MODE == 0 ? (half_n >> 7) + n_tile : nb0;
      const float* sb0 = p.b_scales + ((size_t)e * p.NBw + nb0) * p.KB;
      const float* sb1 = p.b_scales + ((size_t)e * p.NBw + nb1) * p.KB;
      const float sb0_lo = lane < p.KB ? __ldg(sb0 + lane) : 0.f;
      const float sb0_hi = lane + 32 < p.KB ? __ldg(sb0 + lane + 32) : 0.f;
      const float sb1_lo = lane < p.KB ? __ldg(sb1 + lane) : 0.f;
      const float sb1_hi = lane + 32 < p.KB ? __ldg(sb1 + lane + 32) : 0.f;

      // c[i] holds columns (2i, 2i+1) of this thread's 128; promotion uses the packed fp32x2 FMA.
      float2 c[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) c[i] = make_float2(0.f, 0.f);
      bool ok = true;
      for (int kb = 0; kb < p.KB; ++kb, ++it) {
        // every lane polls: one polling lane plus a broadcast measured 136 clk slower per K block
        if (!sm100::mbar_wait(&ctl.tmem_full[acc], acc_phase, abort_flag, p.status, kWaitTmemFull)) { ok = false; break; }
        sm100::tc_fence_after_sync();
        const float s_a = ctl.sa_ring[it & (kScaleSlots - 1)][row];
        const float b0 = __shfl_sync(0xffffffffu, kb < 32 ? sb0_lo : sb0_hi, kb & 31);
        const float b1 = __shfl_sync(0xffffffffu, kb < 32 ? sb1_lo : sb1_hi, kb & 31);
        const float s0 = s_a * b0, s1 = s_a * b1;
        const uint32_t tbase = lane_base + acc * kAccCols;
        // 4 chunks of 32 columns in two rounds: tcgen05.wait::ld drains every outstanding load, so
        // the loads of a round are issued together (64 staging registers) and share one latency.
        {
          uint32_t t0[32], t1[32];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            sm100::tmem_ld_32x32(tbase + chunk_col<MODE>(2 * half, g), t0);
            sm100::tmem_ld_32x32(tbase + chunk_col<MODE>(2 * half + 1, g), t1);
            sm100::tmem_ld_wait();
            const float s = half == 0 ? s0 : s1;
            const float2 s2 = make_float2(s, s);
#pragma unroll
            for (int i = 0; i < 16; ++i)
              c[half * 32 + i] = __ffma2_rn(make_float2(__uint_as_float(t0[2 * i]), __uint_as_float(t0[2 * i + 1])),
                                            s2, c[half * 32 + i]);
#pragma unroll
            for (int i = 0; i < 16; ++i)
              c[half * 32 + 16 + i] = __ffma2_rn(make_float2(__uint_as_float(t1[2 * i]), __uint_as_float(t1[2 * i + 1])),
                                                 s2, c[half * 32 + 16 + i]);
          }
        }
        sm100::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(&ctl.tmem_empty[acc]);
        acc ^= 1; if (acc == 0) acc_phase ^= 1;
      }
      if (!ok) break;

      // Both rendezvous points are used once per tile, so their phase is the tile parity.
      const uint32_t epi_phase = tile_iter & 1;
      const bool issuer = (warp == 4 && lane == 0);
      // The previous tile's TMA stores must have finished reading the staging tile.
      if (issuer) sm100::tma_store_wait_read();
      float amax = 0.f;
      if (MODE == 0) {
        // c[0..31] = gate, c[32..63] = up (float2 each), columns 64g .. 64g+63 of the h block
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float2 gate = c[i], up = c[32 + i];
          float2 h;
          h.x = __fdividef(gate.x, 1.f + __expf(-gate.x)) * up.x;
          h.y = __fdividef(gate.y, 1.f + __expf(-gate.y)) * up.y;
          c[i] = h;
          amax = fmaxf(amax, fmaxf(fabsf(h.x), fabsf(h.y)));
        }
        ctl.amax[epi_phase][g][row] = amax;
      }
      sm100::mbar_arrive(&ctl.epi_bar[0]);
      if (!sm100::mbar_wait(&ctl.epi_bar[0], epi_phase, abort_flag, p.status, kWaitEpilogue)) break;
      // 16-byte chunk `ch` of row `row` inside a 128-byte-wide swizzled sub-tile
      uint8_t* my_row = out_stage + row * 128;
      const int sw = row & 7;
      if (MODE == 0) {
        amax = fmaxf(amax, ctl.amax[epi_phase][g ^ 1][row]);
        const float scale = __fdiv_rn(fmaxf(amax, 1e-4f), 448.f);
        const float inv = __fdividef(1.f, scale);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 q;
          uint32_t* qw = &q.x;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 lo = c[8 * v + 2 * j], hi = c[8 * v + 2 * j + 1];
            qw[j] = pack4_e4m3(lo.x * inv, lo.y * inv, hi.x * inv, hi.y * inv);
          }
          *reinterpret_cast<uint4*>(my_row + (((4 * g + v) ^ sw) << 4)) = q;
        }
        if (g == 0) p.out_scales_t[(size_t)n_tile * p.ld_rows + grow] = scale;
      } else {
        // 256 bf16 columns = 4 sub-tiles of 64 columns (128 bytes); this thread fills sub-tiles 2g, 2g+1
#pragma unroll
        for (int v = 0; v < 16; ++v) {
          uint4 o;
          o.x = pack2_bf16(c[4 * v + 0].x, c[4 * v + 0].y);
          o.y = pack2_bf16(c[4 * v + 1].x, c[4 * v + 1].y);
          o.z = pack2_bf16(c[4 * v + 2].x, c[4 * v + 2].y);
          o.w = pack2_bf16(c[4 * v + 3].x, c[4 * v + 3].y);
          *reinterpret_cast<uint4*>(my_row + (2 * g + (v >> 3)) * (128 * 128) + (((v & 7) ^ sw) << 4)) = o;
        }
      }
      sm100::fence_proxy_async();
      sm100::mbar_arrive(&ctl.epi_bar[1]);
      if (!sm100::mbar_wait(&ctl.epi_bar[1], epi_phase, abort_flag, p.status, kWaitEpilogue)) break;
      if (issuer) {
        if (MODE == 0) {
          sm100::tma_store_2d(&tmap_out, out_stage, n_tile * 128, m_tile * kBM);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            sm100::tma_store_2d(&tmap_out, out_stage + j * (128 * 128), n_tile * 256 + j * 64, m_tile * kBM);
        }
        sm100::tma_store_commit();
      }
    }
    if (warp == 4 && lane == 0) sm100::tma_store_wait_all();   // global writes done before the CTA exits
  }

  // ---------------------------------------------------------------- teardown
  sm100::tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    sm100::tc_fence_after_sync();
    sm100::tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int MODE>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tout, const GemmParams& p, int grid,
           cudaStream_t stream) {
  if (!cab::ensure_dynamic_smem<&moe_gemm_fp8_kernel<MODE>>(smem_bytes<MODE>())) return CAB_ERR_LAUNCH;
  moe_gemm_fp8_kernel<MODE><<<grid, kThreads, smem_bytes<MODE>(), stream>>>(ta, tb, tout, p);
  return cab::launch_status();
}

}  // namespace

extern "C" int moe_grouped_gemm_fp8_launcher(int mode, void* out, float* out_scales_t, const cab_e4m3* a_q,
                                             const float* a_scales_t, const cab_e4m3* w_q,
                                             const float* w_scales, const int* tile_expert,
                                             const int* num_tiles, int max_m_tiles, int rows_cap, int ld_rows,
                                             int E, int N, int K, int* status, int config,
                                             cudaStream_t stream) {
  if (mode != 0 && mode != 1) return CAB_ERR_BAD_ARGUMENT;
  if (!out || !a_q || !a_scales_t || !w_q || !w_scales || (mode == 0 && !out_scales_t)) return CAB_ERR_BAD_ARGUMENT;
  if (max_m_tiles <= 0 || E <= 0 || N <= 0 || K <= 0 || K % 128 != 0) return CAB_ERR_BAD_ARGUMENT;
  if (K > 64 * 128) return CAB_ERR_TOO_LARGE;                 // weight scales of a tile live in two registers per lane
  if (ld_rows % 4 != 0 || !cab::aligned_to(a_scales_t, 16)) return CAB_ERR_MISALIGNED;   // bulk copies of 128 scales
  if (mode == 0 ? N % 128 != 0 : N % 256 != 0) return CAB_ERR_BAD_ARGUMENT;
  if (rows_cap < max_m_tiles * kBM || ld_rows < rows_cap) return CAB_ERR_BAD_ARGUMENT;
  if ((tile_expert == nullptr) != (num_tiles == nullptr)) return CAB_ERR_BAD_ARGUMENT;
  if (!tile_expert && E != 1) return CAB_ERR_BAD_ARGUMENT;
  if (!cab::aligned_to(out, 16) || !cab::aligned_to(a_q, 16) || !cab::aligned_to(w_q, 16)) return CAB_ERR_MISALIGNED;
  const int Nw = mode == 0 ? 2 * N : N;
  if ((long long)E * Nw > 0x7fffffffLL) return CAB_ERR_TOO_LARGE;

  CUtensorMap ta, tb, tout;
  if (!sm100::make_tmap_2d_sw128(&ta, a_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)rows_cap, (uint64_t)K, kBM, kBK) ||
      !sm100::make_tmap_2d_sw128(&tb, w_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)E * Nw, (uint64_t)K, 128, kBK))
    return CAB_ERR_LAUNCH;
  const bool out_ok = mode == 0
      ? sm100::make_tmap_2d_sw128(&tout, out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)rows_cap, (uint64_t)N, kBM, 128)
      : sm100::make_tmap_2d_sw128(&tout, out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)rows_cap, (uint64_t)N, kBM, 64);
  if (!out_ok) return CAB_ERR_LAUNCH;

  GemmParams p;
  p.a_scales_t = a_scales_t; p.b_scales = w_scales; p.tile_expert = tile_expert; p.num_tiles = num_tiles;
  p.fixed_tiles = max_m_tiles; p.KB = K / 128; p.NBw = Nw / 128; p.Nw = Nw;
  p.n_tiles = mode == 0 ? N / 128 : N / 256; p.ld_rows = ld_rows; p.out_ld = N; p.out = out;
  p.out_scales_t = out_scales_t; p.status = status; 
  if (status && cudaMemsetAsync(status, 0, sizeof(int), stream) != cudaSuccess) return CAB_ERR_LAUNCH;
  int grid = cab::kNumSMs;
  if (config > 0) grid = config;                      // tuning: persistent CTAs to launch
  const long long max_total = (long long)max_m_tiles * p.n_tiles;
  if (grid > max_total) grid = (int)max_total;
  return mode == 0 ? launch<0>(ta, tb, tout, p, grid, stream) : launch<1>(ta, tb, tout, p, grid, stream);
}
