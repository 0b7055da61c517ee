// Gated DeltaNet single-step decode for sm_100a.
//
// Per (batch b, value head hv) the recurrent state S is a 128x128 fp32 matrix
// (row i = value channel, column j = key channel). One decode step is
//     alpha = exp(g);  u = S k;  S' = alpha*S + beta*(v - alpha*u) k^T;  o = S' q / sqrt(128)
// Every row of S' depends only on the same row of S, so the step is a single
// streaming pass: a warp owns a row (32 lanes x float4 = 128 columns), forms the
// two dot products S_i.k and S_i.q from the registers it just loaded, and writes
//     S'_i = alpha*S_i + c_i*k,   o_i = (alpha*(S_i.q) + c_i*(k.q)) / sqrt(128),
//     c_i = beta*(v_i - alpha*(S_i.k)).
// Each state element is read once and written once (in place); there is no
// shared memory, no tensor-core work and no second pass. The kernel is bound by
// HBM bandwidth: 2*64 KiB of state traffic per (b, hv) against ~0.1 MFLOP.
//
// Launch shape: one CTA of 8 warps per (b, hv); a warp walks 16 rows. The default kernel
// (gdn_decode_v8_kernel) gives a half-warp one row (16 lanes x 8 floats, 256-bit loads and stores) and
// keeps 16 rows per warp in flight; gdn_decode_kernel is the 128-bit form (a warp per row, ROWS rows in
// flight), kept for states that are not 32-byte aligned and as a tuning reference.
#include "cab_common.cuh"

namespace {

constexpr int kD = 128;           // dk == dv == 128
constexpr int kWarpsPerCta = 8;
constexpr int kRowsPerWarp = kD / kWarpsPerCta;

template <int ROWS>
__global__ void __launch_bounds__(kWarpsPerCta * cab::kWarp)
gdn_decode_kernel(float* __restrict__ state, float* __restrict__ out,
                  const uint2* __restrict__ q, const uint2* __restrict__ k,
                  const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
                  const float* __restrict__ beta, int Hq, int Hv, int group) {
  const int unit = blockIdx.x;  // b * Hv + hv
  const int b = unit / Hv;
  const int hv = unit - b * Hv;
  const int qk_unit = b * Hq + hv / group;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  // Lane l holds columns 4l..4l+3 of k and q (4 bf16 = one 8-byte load).
  const uint2 kraw = __ldg(k + qk_unit * (kD / 4) + lane);
  const uint2 qraw = __ldg(q + qk_unit * (kD / 4) + lane);
  const float k0 = cab::bf16_lo(kraw.x), k1 = cab::bf16_hi(kraw.x);
  const float k2 = cab::bf16_lo(kraw.y), k3 = cab::bf16_hi(kraw.y);
  const float q0 = cab::bf16_lo(qraw.x), q1 = cab::bf16_hi(qraw.x);
  const float q2 = cab::bf16_lo(qraw.y), q3 = cab::bf16_hi(qraw.y);
  const float kq = cab::warp_sum(k0 * q0 + k1 * q1 + k2 * q2 + k3 * q3);

  const float alpha = expf(__ldg(g + unit));
  const float bt = __ldg(beta + unit);
  const float inv_sqrt_d = 0.08838834764831845f;  // 1/sqrt(128)

  const int row_base = warp * kRowsPerWarp;
  float4* srow = reinterpret_cast<float4*>(state) + (size_t)unit * (kD * kD / 4) +
                 (size_t)row_base * (kD / 4) + lane;
  const __nv_bfloat16* vrow = v + (size_t)unit * kD + row_base;
  float* orow = out + (size_t)unit * kD + row_base;

#pragma unroll 1
  for (int it = 0; it < kRowsPerWarp / ROWS; ++it) {
    float4 s[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) s[r] = cab::ld_stream(srow + (it * ROWS + r) * (kD / 4));
    // Without this barrier ptxas sinks each load down to its first use and the
    // warp ends up with one or two loads in flight instead of ROWS.
    __syncwarp();

    float uk[ROWS], uq[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      uk[r] = s[r].x * k0 + s[r].y * k1 + s[r].z * k2 + s[r].w * k3;
      uq[r] = s[r].x * q0 + s[r].y * q1 + s[r].z * q2 + s[r].w * q3;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        uk[r] += __shfl_xor_sync(0xffffffffu, uk[r], off);
        uq[r] += __shfl_xor_sync(0xffffffffu, uq[r], off);
      }
    }

    float o_mine = 0.f;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float vi = __bfloat162float(vrow[it * ROWS + r]);  // warp-uniform address
      const float c = bt * (vi - alpha * uk[r]);
      float4 t;
      t.x = alpha * s[r].x + c * k0;
      t.y = alpha * s[r].y + c * k1;
      t.z = alpha * s[r].z + c * k2;
      t.w = alpha * s[r].w + c * k3;
      cab::st_stream(srow + (it * ROWS + r) * (kD / 4), t);
      const float o = (alpha * uq[r] + c * kq) * inv_sqrt_d;
      if (lane == r) o_mine = o;
    }
    if (lane < ROWS) orow[it * ROWS + lane] = o_mine;
  }
}

// Variant with 256-bit accesses: a half-warp owns a row (16 lanes x 8 floats), a warp works on PAIRS row
// pairs at a time. Same arithmetic per element as the kernel above, but the dot products are reduced over
// 16 lanes (4 shuffle steps for two rows instead of 5 per row), so results can differ in the last bits.
__device__ __forceinline__ void ld_stream8(const float* p, float (&v)[8]) {
  asm volatile("ld.global.cs.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
               : "l"(p));
}
__device__ __forceinline__ void st_stream8(float* p, const float (&v)[8]) {
  asm volatile("st.global.cs.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               :
               : "l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}

template <int PAIRS>
__global__ void __launch_bounds__(kWarpsPerCta * cab::kWarp)
gdn_decode_v8_kernel(float* __restrict__ state, float* __restrict__ out, const uint4* __restrict__ q,
                     const uint4* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                     const float* __restrict__ g, const float* __restrict__ beta, int Hq, int Hv, int group,
                     int reverse) {
  // CTAs start roughly in blockIdx order; `reverse` walks the (b, hv) units from the last to the first. A decode
  // loop that alternates the direction starts every step with the units the previous step wrote last, of which
  // about 80 MB are still in L2 (measured: 946 MB of DRAM traffic per step instead of 1081 MB).
  const int unit = reverse ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
  const int b = unit / Hv;
  const int hv = unit - b * Hv;
  const int qk_unit = b * Hq + hv / group;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int l16 = lane & 15, half = lane >> 4;

  const uint4 kraw = __ldg(k + qk_unit * (kD / 8) + l16);
  const uint4 qraw = __ldg(q + qk_unit * (kD / 8) + l16);
  const float kk[8] = {cab::bf16_lo(kraw.x), cab::bf16_hi(kraw.x), cab::bf16_lo(kraw.y), cab::bf16_hi(kraw.y),
                       cab::bf16_lo(kraw.z), cab::bf16_hi(kraw.z), cab::bf16_lo(kraw.w), cab::bf16_hi(kraw.w)};
  const float qq[8] = {cab::bf16_lo(qraw.x), cab::bf16_hi(qraw.x), cab::bf16_lo(qraw.y), cab::bf16_hi(qraw.y),
                       cab::bf16_lo(qraw.z), cab::bf16_hi(qraw.z), cab::bf16_lo(qraw.w), cab::bf16_hi(qraw.w)};
  float kq = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) kq += kk[i] * qq[i];
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) kq += __shfl_xor_sync(0xffffffffu, kq, off);

  const float alpha = expf(__ldg(g + unit));
  const float bt = __ldg(beta + unit);
  const float inv_sqrt_d = 0.08838834764831845f;
  const int row_base = warp * kRowsPerWarp;
  float* sbase = state + (size_t)unit * (kD * kD) + l16 * 8;
  const __nv_bfloat16* vrow = v + (size_t)unit * kD;
  float* orow = out + (size_t)unit * kD;

#pragma unroll 1
  for (int it = 0; it < kRowsPerWarp / 2 / PAIRS; ++it) {
    float s[PAIRS][8];
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) ld_stream8(sbase + (size_t)(row_base + (it * PAIRS + p) * 2 + half) * kD, s[p]);
    __syncwarp();   // keeps all PAIRS loads in flight (see the kernel above)
    float uk[PAIRS], uq[PAIRS];
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      uk[p] = 0.f; uq[p] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { uk[p] += s[p][i] * kk[i]; uq[p] += s[p][i] * qq[i]; }
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1)
#pragma unroll
      for (int p = 0; p < PAIRS; ++p) {
        uk[p] += __shfl_xor_sync(0xffffffffu, uk[p], off);
        uq[p] += __shfl_xor_sync(0xffffffffu, uq[p], off);
      }
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      const int row = row_base + (it * PAIRS + p) * 2 + half;
      const float vi = __bfloat162float(vrow[row]);
      const float c = bt * (vi - alpha * uk[p]);
      float t[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) t[i] = alpha * s[p][i] + c * kk[i];
      st_stream8(sbase + (size_t)row * kD, t);
      if (l16 == 0) orow[row] = (alpha * uq[p] + c * kq) * inv_sqrt_d;
    }
  }
}

template <int ROWS>
int launch(float* state, float* out, const cab_bf16* q, const cab_bf16* k, const cab_bf16* v,
           const float* g, const float* beta, int B, int Hq, int Hv, cudaStream_t stream) {
  static_assert(kRowsPerWarp % ROWS == 0, "ROWS must divide the rows a warp owns");
  const unsigned grid = static_cast<unsigned>(B) * static_cast<unsigned>(Hv);
  gdn_decode_kernel<ROWS><<<grid, kWarpsPerCta * cab::kWarp, 0, stream>>>(
      state, out, reinterpret_cast<const uint2*>(q), reinterpret_cast<const uint2*>(k),
      reinterpret_cast<const __nv_bfloat16*>(v), g, beta, Hq, Hv, Hv / Hq);
  return cab::launch_status();
}

}  // namespace

extern "C" int gdn_decode_launcher(float* state, float* out, const cab_bf16* q, const cab_bf16* k,
                                   const cab_bf16* v, const float* g, const float* beta, int B,
                                   int Hq, int Hv, int config, cudaStream_t stream) {
  if (B == 0) return CAB_OK;
  if (!state || !out || !q || !k || !v || !g || !beta) return CAB_ERR_BAD_ARGUMENT;
  if (B < 0 || Hq <= 0 || Hv <= 0 || Hv % Hq != 0) return CAB_ERR_BAD_ARGUMENT;
  if ((long long)B * Hv > 0x7fffffffLL) return CAB_ERR_TOO_LARGE;
  if (!cab::aligned_to(state, 16) || !cab::aligned_to(out, 16) || !cab::aligned_to(q, 8) ||
      !cab::aligned_to(k, 8) || !cab::aligned_to(v, 2))
    return CAB_ERR_MISALIGNED;
  // config bit 4 (16): walk the (b, hv) units from the last to the first (256-bit kernels). A caller that flips
  // it from step to step of a decode loop starts every step on the rows the previous step wrote last, which
  // are still in L2; a single step computes the same thing either way. The low four bits choose the kernel
  // form: 0 (default) and 3 use 256-bit accesses (half-warp per row); they need a 32-byte aligned state and
  // 16-byte aligned q/k, otherwise the 128-bit kernel with the same amount in flight takes over.
  const int reverse = (config >= 0 && (config & 16)) ? 1 : 0;
  if (config >= 0) config &= 15;
  const bool v8_ok = cab::aligned_to(state, 32) && cab::aligned_to(q, 16) && cab::aligned_to(k, 16);
  if ((config == 3 || config < 1 || config > 4) && v8_ok) {
    const unsigned grid = static_cast<unsigned>(B) * static_cast<unsigned>(Hv);
    const uint4* q4 = reinterpret_cast<const uint4*>(q);
    const uint4* k4 = reinterpret_cast<const uint4*>(k);
    const __nv_bfloat16* vb = reinterpret_cast<const __nv_bfloat16*>(v);
    if (config == 3)
      gdn_decode_v8_kernel<4><<<grid, kWarpsPerCta * cab::kWarp, 0, stream>>>(state, out, q4, k4, vb, g, beta, Hq, Hv, Hv / Hq, reverse);
    else
      gdn_decode_v8_kernel<8><<<grid, kWarpsPerCta * cab::kWarp, 0, stream>>>(state, out, q4, k4, vb, g, beta, Hq, Hv, Hv / Hq, reverse);
    return cab::launch_status();
  }
  switch (config) {
    case 1: return launch<4>(state, out, q, k, v, g, beta, B, Hq, Hv, stream);
    case 2: return launch<16>(state, out, q, k, v, g, beta, B, Hq, Hv, stream);
    default: return launch<8>(state, out, q, k, v, g, beta, B, Hq, Hv, stream);
  }
}
