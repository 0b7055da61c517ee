// MoE routing for sm_100a: router logits and the two top-k rules.
//
//   moe_router_logits   logits[t, e] = sum_h x[t, h] * wr[e, h]   bf16 in, fp32 out
//   moe_route_softmax   k largest logits per token (descending, ties -> lower
//                       expert id) and the softmax over just those k
//   moe_route_sigmoid   DeepSeek-V3 style: s = sigmoid(logit), c = s + bias, keep the
//                       best `topk_group` of `n_group` expert groups (group score =
//                       sum of its two largest c), then the k largest c inside them;
//                       weights s[idx] / sum(s[idx]) * scale
//
// Index outputs are meant to be bit-identical to a CPU statement of the same
// rules, so every comparison that decides an index uses only values that are
// reproducible bit for bit: raw fp32 logits for the softmax rule, and for the
// sigmoid rule a sigmoid evaluated in fp64 and rounded once to fp32 followed by
// IEEE fp32 adds (no fast-math approximations on that path).
//
// The selection kernels run one warp per token with the token's E <= 256 scores
// spread over the lanes (expert e lives in lane e % 32, slot e / 32).
#include "cab_common.cuh"
#include "sm100_primitives.cuh"

namespace {

constexpr int kMaxE = 256;
constexpr int kSlots = kMaxE / 32;
constexpr int kMaxTopK = 32;

// ------------------------------------------------------------------ logits
// A warp computes 16-token row tiles x (up to) 64 experts per pass with mma.sync
// m16n8k16 bf16 (fp32 accumulate). Fragments come straight from global memory:
// a lane reads 16 contiguous bytes (8 bf16) of its A rows and of its B row and
// feeds them to two MMAs. That assigns the k index inside a 32-wide chunk in a
// permuted order, identically for A and B, which a dot product does not notice.
__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1,
                                                 uint32_t a2, uint32_t a3, uint32_t b0,
                                                 uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// CTA = 8 warps on MT*16 tokens and (per pass) 64 experts; warp w sums the k range
// [w*H/8, (w+1)*H/8) (split-K inside the CTA, so that T/16 row tiles still fill the GPU and every
// warp has many independent 16-byte loads in flight); the 8 partial tiles are added in warp order
// through shared memory, which keeps the result independent of scheduling.
template <int MT>
__global__ void __launch_bounds__(256)
router_logits_kernel(float* __restrict__ logits, const __nv_bfloat16* __restrict__ x,
                     const __nv_bfloat16* __restrict__ wr, int T, int H, int E) {
  __shared__ float part[8][16][64 + 1];   // one 16-token row tile at a time
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t0 = blockIdx.x * (MT * 16);
  const int r = lane >> 2;          // fragment row within 8
  const int kq = (lane & 3) * 8;    // this lane's 8 consecutive k inside a 32-chunk
  const int kchunks = H / 32;
  const int c_begin = (kchunks * warp) / 8, c_end = (kchunks * (warp + 1)) / 8;
  const uint4* xa[MT];
  const uint4* xb[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    xa[m] = reinterpret_cast<const uint4*>(x + (size_t)min(t0 + m * 16 + r, T - 1) * H + kq);
    xb[m] = reinterpret_cast<const uint4*>(x + (size_t)min(t0 + m * 16 + r + 8, T - 1) * H + kq);
  }
  for (int e0 = 0; e0 < E; e0 += 64) {
    const int ntiles = min(8, (E - e0) >> 3);
    float acc[MT][8][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[m][j][0] = acc[m][j][1] = acc[m][j][2] = acc[m][j][3] = 0.f;
    const __nv_bfloat16* wbase = wr + (size_t)(e0 + r) * H + kq;
#pragma unroll 2
    for (int c = c_begin; c < c_end; ++c) {
      uint4 a_lo[MT], a_hi[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) { a_lo[m] = __ldg(xa[m] + c * 4); a_hi[m] = __ldg(xb[m] + c * 4); }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < ntiles) {
          const uint4 b = __ldg(reinterpret_cast<const uint4*>(wbase + (size_t)j * 8 * H + c * 32));
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            mma_bf16_16x8x16(acc[m][j], a_lo[m].x, a_hi[m].x, a_lo[m].y, a_hi[m].y, b.x, b.y);
            mma_bf16_16x8x16(acc[m][j], a_lo[m].z, a_hi[m].z, a_lo[m].w, a_hi[m].w, b.z, b.w);
          }
        }
      }
    }
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        part[warp][r][j * 8 + col] = acc[m][j][0];
        part[warp][r][j * 8 + col + 1] = acc[m][j][1];
        part[warp][r + 8][j * 8 + col] = acc[m][j][2];
        part[warp][r + 8][j * 8 + col + 1] = acc[m][j][3];
      }
      __syncthreads();
      for (int i = threadIdx.x; i < 16 * 64; i += 256) {
        const int row = i >> 6, e = i & 63;
        const int t = t0 + m * 16 + row;
        if (t < T && e < ntiles * 8) {
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < 8; ++w) sum += part[w][row][e];
          logits[(size_t)t * E + e0 + e] = sum;
        }
      }
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------ logits on tcgen05
// The same product for large batches: a CTA takes 128 tokens and all E experts (E a multiple of 32, at most
// 256), TMA brings 128 x 64 bf16 of x and E x 64 of the router weight per stage (128-byte swizzle), one thread
// issues tcgen05.mma kind::f16 (M 128, N E, K 16) into a single fp32 accumulator in tensor memory that runs over
// the whole of H, and four warps write the rows out. One accumulation chain in k order per (token, expert), so
// the result does not depend on scheduling.
constexpr int kTcStages = 4;
struct __align__(16) TcControl {
  uint64_t full[kTcStages], empty[kTcStages], acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(192, 1)
router_logits_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                        float* __restrict__ logits, int T, int H, int E, uint32_t tmem_cols) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = 128 * 128 + E * 128;
  TcControl& ctl = *reinterpret_cast<TcControl*>(tiles + kTcStages * stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * 128;
  const int ksteps = H / 64;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcStages; ++s) { sm100::mbar_init(&ctl.full[s], 1); sm100::mbar_init(&ctl.empty[s], 1); }
    sm100::mbar_init(&ctl.acc_full, 1);
    ctl.abort_flag = 0;
    sm100::mbar_fence_init();
    sm100::prefetch_tensormap(&tmap_x);
    sm100::prefetch_tensormap(&tmap_w);
  }
  if (warp == 1) {
    sm100::tmem_alloc(&ctl.tmem_base, tmem_cols);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before_sync();
  __syncthreads();
  sm100::tc_fence_after_sync();
  const uint32_t tmem_base = ctl.tmem_base;
  volatile int* abort_flag = &ctl.abort_flag;

  if (warp == 0 && lane == 0) {
    int stage = 0; uint32_t phase = 0;
    for (int ks = 0; ks < ksteps; ++ks) {
      if (!sm100::mbar_wait(&ctl.empty[stage], phase ^ 1, abort_flag, nullptr, 0)) break;
      uint8_t* dst = tiles + stage * stage_bytes;
      sm100::mbar_arrive_expect_tx(&ctl.full[stage], stage_bytes);
      sm100::tma_load_2d(dst, &tmap_x, &ctl.full[stage], ks * 64, m0);
      sm100::tma_load_2d(dst + 128 * 128, &tmap_w, &ctl.full[stage], ks * 64, 0);
      if (++stage == kTcStages) { stage = 0; phase ^= 1; }
    }
  } else if (warp == 1 && lane == 0) {
    const uint32_t idesc = sm100::umma_idesc(1 /* bf16 */, 128, E);
    int stage = 0; uint32_t phase = 0;
    bool ok = true;
    for (int ks = 0; ks < ksteps; ++ks) {
      if (!sm100::mbar_wait(&ctl.full[stage], phase, abort_flag, nullptr, 0)) { ok = false; break; }
      sm100::tc_fence_after_sync();
      const uint32_t a_addr = sm100::smem_u32(tiles + stage * stage_bytes);
      const uint64_t a_desc = sm100::umma_desc_k_sw128(a_addr);
      const uint64_t b_desc = sm100::umma_desc_k_sw128(a_addr + 128 * 128);
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4)   // 16 bf16 = 32 bytes of K per instruction: +2 in 16-byte units
        sm100::umma_f16(tmem_base, a_desc + 2 * k4, b_desc + 2 * k4, idesc, (ks > 0 || k4 > 0) ? 1u : 0u);
      sm100::umma_commit(&ctl.empty[stage]);
      if (++stage == kTcStages) { stage = 0; phase ^= 1; }
    }
    if (ok) sm100::umma_commit(&ctl.acc_full);
  } else if (warp >= 2) {
    const int quad = warp & 3;                       // the TMEM lane quadrant a warp may read is warp id % 4
    const int t = m0 + quad * 32 + lane;
    if (sm100::mbar_wait(&ctl.acc_full, 0, abort_flag, nullptr, 0)) {
      sm100::tc_fence_after_sync();
      const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
      for (int c = 0; c < E; c += 32) {
        uint32_t v[32];
        sm100::tmem_ld_32x32(lane_base + c, v);
        sm100::tmem_ld_wait();
        if (t < T) {
          float4* dst = reinterpret_cast<float4*>(logits + (size_t)t * E + c);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2]),
                                 __uint_as_float(v[4 * i + 3]));
        }
      }
    }
  }
  sm100::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after_sync();
    sm100::tmem_dealloc(tmem_base, tmem_cols);
  }
}

// Launches the tensor-core form when the shapes fit it; returns false when the caller should use the other kernel.
bool launch_router_logits_tc(float* logits, const cab_bf16* x, const cab_bf16* wr, int T, int H, int E,
                             cudaStream_t stream, int& rc) {
  if (T < 512 || E % 32 != 0 || E > 256 || H % 64 != 0 || !cab::aligned_to(logits, 16)) return false;
  CUtensorMap tx, tw;
  if (!sm100::make_tmap_2d_sw128(&tx, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)T, (uint64_t)H, 128, 64) ||
      !sm100::make_tmap_2d_sw128(&tw, wr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)E, (uint64_t)H, (uint32_t)E, 64))
    return false;
  const int smem = kTcStages * (128 * 128 + E * 128) + (int)sizeof(TcControl) + 1024;
  if (!cab::ensure_dynamic_smem<&router_logits_tc_kernel>(kTcStages * (128 * 128 + 256 * 128) + (int)sizeof(TcControl) + 1024)) {
    rc = CAB_ERR_LAUNCH;
    return true;
  }
  uint32_t cols = 32;
  while ((int)cols < E) cols <<= 1;
  router_logits_tc_kernel<<<(T + 127) / 128, 192, smem, stream>>>(tx, tw, logits, T, H, E, cols);
  rc = cab::launch_status();
  return true;
}

// ------------------------------------------------------------------ selection
// (value, index) ordering used everywhere: larger value first, equal values ->
// smaller index first.
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

// Picks the best remaining entry of the warp-distributed array `val` (slot j of
// lane l is entry j*32+l; entries whose bit is set in `taken` are skipped, as are
// entries >= n). Every lane returns the same (value, index); index -1 if none is left.
__device__ __forceinline__ void warp_argbest(const float (&val)[kSlots], uint32_t taken, int n,
                                             int lane, float& best_v, int& best_i) {
  float bv = -INFINITY;
  int bi = 0x7fffffff;
#pragma unroll
  for (int j = 0; j < kSlots; ++j) {
    const int e = j * 32 + lane;
    if (e < n && !((taken >> j) & 1u) && better(val[j], e, bv, bi)) { bv = val[j]; bi = e; }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  best_v = bv;
  best_i = (bi == 0x7fffffff) ? -1 : bi;
}

__global__ void __launch_bounds__(256)
route_softmax_topk_kernel(int* __restrict__ topk_idx, float* __restrict__ topk_w,
                          const float* __restrict__ logits, int T, int E, int k) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  float val[kSlots];
#pragma unroll
  for (int j = 0; j < kSlots; ++j) {
    const int e = j * 32 + lane;
    val[j] = e < E ? __ldg(logits + (size_t)t * E + e) : -INFINITY;
  }
  uint32_t taken = 0;
  float my_v = 0.f, top_v = 0.f, denom = 0.f;
  int my_i = 0;
  for (int s = 0; s < k; ++s) {
    float bv; int bi;
    warp_argbest(val, taken, E, lane, bv, bi);
    if (bi >= 0 && (bi & 31) == lane) taken |= 1u << (bi >> 5);
    if (s == 0) top_v = bv;
    const float p = expf(bv - top_v);
    denom += p;
    if (lane == s) { my_v = p; my_i = bi; }
  }
  if (lane < k) {
    topk_idx[(size_t)t * k + lane] = my_i;
    topk_w[(size_t)t * k + lane] = __fdividef(my_v, denom);
  }
}

__global__ void __launch_bounds__(256)
route_sigmoid_group_topk_kernel(int* __restrict__ topk_idx, float* __restrict__ topk_w,
                                const float* __restrict__ logits, const float* __restrict__ bias,
                                int T, int E, int k, int n_group, int topk_group, float scale) {
  __shared__ float c_sm[8][kMaxE];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  float s_val[kSlots], c_val[kSlots];
#pragma unroll
  for (int j = 0; j < kSlots; ++j) {
    const int e = j * 32 + lane;
    if (e < E) {
      const double l = (double)__ldg(logits + (size_t)t * E + e);
      s_val[j] = (float)(1.0 / (1.0 + exp(-l)));          // fp64 sigmoid, rounded once
      c_val[j] = __fadd_rn(s_val[j], __ldg(bias + e));
      c_sm[warp][e] = c_val[j];
    } else {
      s_val[j] = 0.f;
      c_val[j] = -INFINITY;
    }
  }
  __syncwarp();
  // group scores: lane g scans group g (n_group <= 32)
  const int gsize = E / n_group;
  float gscore[kSlots];
#pragma unroll
  for (int j = 0; j < kSlots; ++j) gscore[j] = -INFINITY;
  if (lane < n_group) {
    float m1 = -INFINITY, m2 = -INFINITY;
    for (int i = 0; i < gsize; ++i) {
      const float v = c_sm[warp][lane * gsize + i];
      if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
    }
    gscore[0] = gsize >= 2 ? __fadd_rn(m1, m2) : m1;
  }
  uint32_t g_taken = 0, keep_mask = 0;
  for (int s = 0; s < topk_group; ++s) {
    float bv; int bi;
    warp_argbest(gscore, g_taken, n_group, lane, bv, bi);
    if (bi >= 0) {
      keep_mask |= 1u << bi;
      if (bi == lane) g_taken |= 1u;
    }
  }
#pragma unroll
  for (int j = 0; j < kSlots; ++j) {
    const int e = j * 32 + lane;
    if (e < E && !((keep_mask >> (e / gsize)) & 1u)) c_val[j] = -INFINITY;
  }
  uint32_t taken = 0;
  float my_s = 0.f, denom = 0.f;
  int my_i = 0;
  for (int s = 0; s < k; ++s) {
    float bv; int bi;
    warp_argbest(c_val, taken, E, lane, bv, bi);
    float sv = 0.f;
    if (bi >= 0 && (bi & 31) == lane) {
      taken |= 1u << (bi >> 5);
#pragma unroll
      for (int j = 0; j < kSlots; ++j) if (j == (bi >> 5)) sv = s_val[j];
    }
    sv = __shfl_sync(0xffffffffu, sv, bi >= 0 ? (bi & 31) : 0);
    denom += sv;
    if (lane == s) { my_s = sv; my_i = bi; }
  }
  if (lane < k) {
    topk_idx[(size_t)t * k + lane] = my_i;
    topk_w[(size_t)t * k + lane] = __fdiv_rn(my_s, denom) * scale;
  }
}

bool route_args_ok(int T, int E, int k) { return T >= 0 && E > 0 && E <= kMaxE && k > 0 && k <= kMaxTopK && k <= E; }

}  // namespace

extern "C" int moe_router_logits_launcher(float* logits, const cab_bf16* x, const cab_bf16* wr,
                                          int T, int H, int E, int config, cudaStream_t stream) {
  if (T == 0) return CAB_OK;
  if (!logits || !x || !wr) return CAB_ERR_BAD_ARGUMENT;
  if (T < 0 || H <= 0 || E <= 0 || H % 32 != 0 || E % 8 != 0) return CAB_ERR_BAD_ARGUMENT;
  if (!cab::aligned_to(x, 16) || !cab::aligned_to(wr, 16) || !cab::aligned_to(logits, 8))
    return CAB_ERR_MISALIGNED;
  // config 1 keeps the mma.sync kernels for every shape; otherwise large batches go to the tcgen05 kernel
  int rc = CAB_OK;
  if (config != 1 && launch_router_logits_tc(logits, x, wr, T, H, E, stream, rc)) return rc;
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(wr);
  // Every CTA reads the whole router weight, so a large weight (E*H) wants many tokens per CTA: 64
  // (each weight fragment feeds four row tiles) once the weight exceeds 1 MB, else 16.
  if ((size_t)E * H * 2 >= (1u << 20) && T >= 64 * 32)
    router_logits_kernel<4><<<(T + 63) / 64, 256, 0, stream>>>(logits, xp, wp, T, H, E);
  else
    router_logits_kernel<1><<<(T + 15) / 16, 256, 0, stream>>>(logits, xp, wp, T, H, E);
  return cab::launch_status();
}

extern "C" int moe_route_softmax_topk_launcher(int* topk_idx, float* topk_w, const float* logits,
                                               int T, int E, int k, int config, cudaStream_t stream) {
  (void)config;
  if (T == 0) return CAB_OK;
  if (!topk_idx || !topk_w || !logits || !route_args_ok(T, E, k)) return CAB_ERR_BAD_ARGUMENT;
  route_softmax_topk_kernel<<<(T + 7) / 8, 256, 0, stream>>>(topk_idx, topk_w, logits, T, E, k);
  return cab::launch_status();
}

extern "C" int moe_route_sigmoid_group_topk_launcher(int* topk_idx, float* topk_w,
                                                     const float* logits, const float* bias, int T,
                                                     int E, int k, int n_group, int topk_group,
                                                     float routed_scaling_factor, int config,
                                                     cudaStream_t stream) {
  (void)config;
  if (T == 0) return CAB_OK;
  if (!topk_idx || !topk_w || !logits || !bias || !route_args_ok(T, E, k)) return CAB_ERR_BAD_ARGUMENT;
  if (n_group <= 0 || n_group > 32 || E % n_group != 0 || topk_group <= 0 || topk_group > n_group ||
      k > topk_group * (E / n_group))
    return CAB_ERR_BAD_ARGUMENT;
  route_sigmoid_group_topk_kernel<<<(T + 7) / 8, 256, 0, stream>>>(
      topk_idx, topk_w, logits, bias, T, E, k, n_group, topk_group, routed_scaling_factor);
  return cab::launch_status();
}
