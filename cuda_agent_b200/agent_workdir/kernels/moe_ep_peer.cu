// Expert-parallel dispatch and return for the FP8 MoE layer, with the exchange done by the kernels
// themselves over peer memory (NVLink / NVSwitch): no collective library call and no host round trip
// sits between the routing of a token and the grouped GEMMs that serve it.
//
// Every rank owns one "exchange buffer" of fixed capacity, laid out identically on all ranks, and
// maps the buffers of all other ranks (CUDA IPC between processes, plain pointers inside one). With
// R ranks, t_cap tokens per rank at most, nb = H/128, k experts per token:
//
//   recv_rows  [R][t_cap][H]           e4m3   copy p of source rank s lands in row (s, p)
//   recv_side  [R][t_cap][nb + 2k]     32-bit the copy's nb scales, k weights, k local expert ids (-1 = none)
//   recv_flag  [R]                     u64    written last by source s: (call number << 32) | copies sent
//   back_rows  [R][t_cap][H]           bf16   the weighted partial sum rank d computed for my copy (d, p)
//   back_flag  [R]                     u64    written last by rank d: call number << 32
//
// One layer call on a rank (all launches asynchronous on the caller's stream):
//   plan      per destination rank, a scan over the tokens gives every (token, destination) copy its row
//   dispatch  warps quantise a token's row once (1x128 e4m3) and store it, its scales and its
//             (weight, local expert) slots straight into the destination ranks' recv_* rows; a one-warp
//             kernel behind it publishes recv_flag on every peer (release at system scope)
//   receive   one small CTA waits (bounded) for the R flags, then the valid slots become sort keys
//   permute   moe_permute_launcher sorts the keys by local expert into the padded row space
//   gather    received rows are copied into that row space, scales transposed
//   GEMMs     gate/up + SwiGLU + re-quantise, down
//   return    per received copy, sum_j w_j y_j in fp32 -> bf16, stored into the source rank's back_rows;
//             a one-warp kernel behind it publishes back_flag on every peer
//   combine   one small CTA waits (bounded) for the R back flags; out[t] = sum over destinations of the
//             partial rows (+ shared expert)
//
// Why one buffer generation is enough: a rank stores into a peer's recv_* rows for call c+1 only after
// its own combine of call c, which waited for that peer's back_flag of call c, and the peer publishes
// that flag after its last read of the rows of call c. Symmetrically a rank stores into a peer's
// back_rows for call c+1 only after it has seen the peer's recv_flag of call c+1, which the peer
// publishes after its combine of call c has finished reading them.
//
// Every wait on a flag is bounded (kFlagWaitCycles); when it runs out the kernel records a code in the
// context's status words, treats the missing rank as having sent nothing and returns.
#include "cab_common.cuh"

#include <cuda_fp8.h>

#include <algorithm>
#include <cstring>
#include <new>

namespace {

constexpr int kMaxWorld = 16;
constexpr int kMaxK = 32;
constexpr long long kFlagWaitCycles = 6000000000LL;   // about three seconds at 1.9 GHz
constexpr float kAmaxFloor = 1e-4f;
constexpr float kFp8Max = 448.f;

struct PeerTable {
  uint8_t* base[kMaxWorld];
};

struct Layout {
  int world, t_cap, H, k, nb, side_ld;
  size_t off_rows, off_side, off_flag, off_back, off_back_flag, bytes;
};

Layout make_layout(int world, int t_cap, int H, int k) {
  Layout L;
  L.world = world; L.t_cap = t_cap; L.H = H; L.k = k; L.nb = H / 128; L.side_ld = L.nb + 2 * k;
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  size_t o = 0;
  L.off_rows = o;      o = up(o + (size_t)world * t_cap * H);
  L.off_side = o;      o = up(o + (size_t)world * t_cap * L.side_ld * 4);
  L.off_flag = o;      o = up(o + (size_t)kMaxWorld * 8);
  L.off_back = o;      o = up(o + (size_t)world * t_cap * H * 2);
  L.off_back_flag = o; o = up(o + (size_t)kMaxWorld * 8);
  L.bytes = o;
  return L;
}

struct Ctx {
  Layout L;
  int rank, device, e_local;
  uint8_t* base;                 // this rank's exchange buffer
  PeerTable peers;               // every rank's buffer as addressable from this device
  bool ipc_opened[kMaxWorld];
  bool connected;
  unsigned epoch;                // layer calls made so far
  // local tables (device memory, sized at creation)
  int* copy_pos;                 // [t_cap][world]  row of token t's copy inside destination d's segment, or -1
  int* back_row;                 // [t_cap][world]  d * t_cap + copy_pos, or -1: rows of back_rows to add up
  int* n_copies;                 // [world]
  int* src_count;                // [world] copies received per source in the current call
  int* keys;                     // [world * t_cap * k]
  float* ones;                   // [t_cap * world]
  int* status;                   // [4] 0: wait for dispatch flags, 1: wait for return flags, 2, 3: spare
  cudaStream_t side_stream;      // the shared expert runs here, beside the exchange
  cudaEvent_t fork_event, join_event;
};

enum { kWaitDispatch = 301, kWaitReturn = 302 };

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

// ------------------------------------------------------------------ plan
// CTA d: which tokens have an expert on rank d, and the rank of each such token among them. A thread owns a
// run of consecutive tokens (at most 32: t_cap <= 32768), remembers which of them go to rank d in a bit mask,
// and after the block scan writes their positions without reading the routing table again.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int* __restrict__ topk_idx, int T, int k, int e_local, int world, int t_cap,
               int* __restrict__ copy_pos, int* __restrict__ back_row, int* __restrict__ n_copies) {
  __shared__ int warp_tot[32];
  const int d = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (T + 1023) / 1024;
  const int t0 = tid * per, t1 = min(T, t0 + per);
  const int lo = d * e_local, hi = lo + e_local;
  uint32_t mask = 0;
  if ((k & 3) == 0) {
    for (int t = t0; t < t1; ++t) {
      const int4* row = reinterpret_cast<const int4*>(topk_idx + (size_t)t * k);
      bool has = false;
      for (int j = 0; j < (k >> 2); ++j) {
        const int4 e = __ldg(row + j);
        has |= (e.x >= lo && e.x < hi) | (e.y >= lo && e.y < hi) | (e.z >= lo && e.z < hi) | (e.w >= lo && e.w < hi);
      }
      mask |= (has ? 1u : 0u) << (t - t0);
    }
  } else {
    for (int t = t0; t < t1; ++t) {
      bool has = false;
      for (int j = 0; j < k; ++j) {
        const int e = __ldg(topk_idx + (size_t)t * k + j);
        has |= (e >= lo && e < hi);
      }
      mask |= (has ? 1u : 0u) << (t - t0);
    }
  }
  const int mine = __popc(mask);
  int inc = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, inc, off);
    if (lane >= off) inc += a;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  int base = 0;
  for (int w = 0; w < warp; ++w) base += warp_tot[w];
  int pos = base + inc - mine;
  for (int t = t0; t < t1; ++t) {
    const bool has = (mask >> (t - t0)) & 1u;
    copy_pos[(size_t)t * world + d] = has ? pos : -1;
    back_row[(size_t)t * world + d] = has ? d * t_cap + pos : -1;
    pos += has ? 1 : 0;
  }
  if (tid == 1023) n_copies[d] = base + inc;
}

// ------------------------------------------------------------------ dispatch
// One warp per token and 1024 columns: 1x128 e4m3 quantisation (the rule of moe_quant_dispatch_kernel) and stores into
// every destination rank's receive rows. ep_publish_kernel, launched behind it, publishes the flags.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx,
                   const float* __restrict__ topk_w, const int* __restrict__ copy_pos,
                   int T, int rank, int e_local,
                   const __grid_constant__ Layout L, const __grid_constant__ PeerTable peers) {
  // a warp per (token, 1024-column segment); the warp of segment 0 also writes the token's side band
  const int lane = threadIdx.x & 31;
  const int H = L.H, k = L.k, world = L.world;
  const int segs = (H + 1023) >> 10;
  // (the CTAs walk the segments with a grid stride: every CTA ends with a system-scope fence and a count,
  // so there are a few per SM, not one per eight segments)
  const long long n_items = (long long)T * segs, stride = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long wi = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); wi < n_items; wi += stride) {
    const int t = (int)(wi / segs);
    const int c0 = (int)(wi - (long long)t * segs) << 10;
    const int my_e = lane < k ? __ldg(topk_idx + (size_t)t * k + lane) : -1;
    const float my_w = lane < k ? __ldg(topk_w + (size_t)t * k + lane) : 0.f;
    const int my_dest = my_e >= 0 ? my_e / e_local : -1;
    const int my_pos = lane < world ? __ldg(copy_pos + (size_t)t * world + lane) : -1;   // lane d: copy for rank d
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
        if (c0 + u * 256 >= H) break;                    // warp-uniform: nothing left of the row
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
        for (int d = 0; d < world; ++d) {
          const int pos = __shfl_sync(0xffffffffu, my_pos, d);
          if (pos < 0 || !live) continue;
          const size_t slot = (size_t)rank * L.t_cap + pos;
          *reinterpret_cast<uint2*>(peers.base[d] + L.off_rows + slot * H + col) = q;
          if ((lane & 15) == 0)
            reinterpret_cast<float*>(peers.base[d] + L.off_side)[slot * L.side_ld + (col >> 7)] = scale;
        }
      }
    }
    // slots of the side band: lane j < k holds entry j of the token
    for (int d = 0; d < world && c0 == 0; ++d) {
      const int pos = __shfl_sync(0xffffffffu, my_pos, d);
      if (pos < 0 || lane >= k) continue;
      const size_t slot = (size_t)rank * L.t_cap + pos;
      uint32_t* side = reinterpret_cast<uint32_t*>(peers.base[d] + L.off_side) + slot * L.side_ld + L.nb;
      const bool here = my_dest == d;
      side[lane] = __float_as_uint(here ? my_w : 0.f);
      side[k + lane] = (uint32_t)(here ? my_e - d * e_local : -1);
    }
  }
}

// ------------------------------------------------------------------ publish
// Runs after the kernel whose stores it announces (stream order: that kernel has completed, its stores to
// this GPU and to the peers have been performed). Thread d writes this rank's flag on rank d, release at
// system scope: (call number << 32) | counts[d], or the call number alone when counts is null.
__global__ void __launch_bounds__(32)
ep_publish_kernel(const __grid_constant__ PeerTable peers, size_t flag_offset, int rank, int world, unsigned epoch,
                  const int* __restrict__ counts) {
  const int d = threadIdx.x;
  if (d >= world) return;
  unsigned long long* flag = reinterpret_cast<unsigned long long*>(peers.base[d] + flag_offset) + rank;
  const unsigned low = counts ? (unsigned)__ldg(counts + d) : 0u;
  st_release_sys_u64(flag, ((unsigned long long)epoch << 32) | low);
}

// ------------------------------------------------------------------ bounded wait for R flags
// Thread s waits until flag[s] carries this call's number; counts[s] (may be null) receives its low word.
__global__ void __launch_bounds__(32)
ep_wait_flags_kernel(const unsigned long long* __restrict__ flags, int world, unsigned epoch, int t_cap,
                     int* __restrict__ counts, int* __restrict__ status, int where) {
  const int s = threadIdx.x;
  if (s >= world) return;
  const long long t0 = clock64();
  unsigned long long v = ld_acquire_sys_u64(flags + s);
  while ((unsigned)(v >> 32) != epoch) {
    if (clock64() - t0 > kFlagWaitCycles) {
      atomicCAS(status, 0, where);
      if (counts) counts[s] = 0;
      return;
    }
    __nanosleep(200);
    v = ld_acquire_sys_u64(flags + s);
  }
  if (counts) counts[s] = min((int)(unsigned)(v & 0xffffffffu), t_cap);
}

// keys[(s * t_cap + p) * k + j] = local expert of slot j of copy (s, p), -1 for an empty slot or a row
// past what source s sent in this call.
__global__ void __launch_bounds__(256)
ep_keys_kernel(const uint32_t* __restrict__ side, const int* __restrict__ src_count, int world, int t_cap, int k,
               int side_ld, int nb, int e_local, int* __restrict__ keys) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)world * t_cap * k;
  if (i >= total) return;
  const int j = (int)(i % k);
  const long long slot = i / k;
  const int s = (int)(slot / t_cap), p = (int)(slot - (long long)s * t_cap);
  int e = -1;
  if (p < __ldg(src_count + s)) {
    e = (int)__ldg(side + slot * side_ld + nb + k + j);
    if (e < 0 || e >= e_local) e = -1;
  }
  keys[i] = e;
}

// Live copy c (0 <= c < sum of src_count) -> (source, row within the source's segment).
__device__ __forceinline__ bool live_copy(int c, const int* __restrict__ src_count, int world, int& s, int& p) {
  int start = 0;
  for (s = 0; s < world; ++s) {
    const int n = __ldg(src_count + s);
    if (c < start + n) { p = c - start; return true; }
    start += n;
  }
  return false;
}

// ------------------------------------------------------------------ gather into the padded row space
__global__ void __launch_bounds__(256)
ep_gather_kernel(uint8_t* __restrict__ a_q, float* __restrict__ a_s_t, const uint8_t* __restrict__ rows,
                 const float* __restrict__ side, const int* __restrict__ src_count, const int* __restrict__ dst_row,
                 int world, int t_cap, int k, int H, int side_ld, int ld_rows) {
  __shared__ int dst[kMaxK];
  for (int c = blockIdx.x;; c += gridDim.x) {
    int s, p;
    if (!live_copy(c, src_count, world, s, p)) return;
    const size_t slot = (size_t)s * t_cap + p;
    __syncthreads();
    if (threadIdx.x < k) dst[threadIdx.x] = __ldg(dst_row + slot * k + threadIdx.x);
    __syncthreads();
    const uint4* src = reinterpret_cast<const uint4*>(rows + slot * H);
    for (int u = threadIdx.x; u < H / 16; u += blockDim.x) {
      const uint4 v = __ldcs(src + u);
      for (int j = 0; j < k; ++j)
        if (dst[j] >= 0) reinterpret_cast<uint4*>(a_q + (size_t)dst[j] * H)[u] = v;
    }
    for (int b = threadIdx.x; b < H / 128; b += blockDim.x) {
      const float sc = __ldg(side + slot * side_ld + b);
      for (int j = 0; j < k; ++j)
        if (dst[j] >= 0) a_s_t[(size_t)b * ld_rows + dst[j]] = sc;
    }
  }
}

// ------------------------------------------------------------------ return
// Per received copy: sum over its slots (ascending) of w_j * y[row_j], fp32 -> bf16, stored into the
// source rank's back_rows; ep_publish_kernel, launched behind it, publishes the flags.
__global__ void __launch_bounds__(256)
ep_return_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ side,
                 const int* __restrict__ src_count, const int* __restrict__ dst_row, int rank,
                 const __grid_constant__ Layout L, const __grid_constant__ PeerTable peers) {
  __shared__ int rows[kMaxK];
  __shared__ float wts[kMaxK];
  const int k = L.k, H = L.H, world = L.world;
  for (int c = blockIdx.x;; c += gridDim.x) {
    int s, p;
    if (!live_copy(c, src_count, world, s, p)) break;
    const size_t slot = (size_t)s * L.t_cap + p;
    __syncthreads();
    if (threadIdx.x < k) {
      rows[threadIdx.x] = __ldg(dst_row + slot * k + threadIdx.x);
      wts[threadIdx.x] = __ldg(side + slot * L.side_ld + L.nb + threadIdx.x);
    }
    __syncthreads();
    uint4* out = reinterpret_cast<uint4*>(peers.base[s] + L.off_back + ((size_t)rank * L.t_cap + p) * H * 2);
    for (int col = threadIdx.x * 8; col < H; col += blockDim.x * 8) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      // slots in batches of eight: the batch's row loads are issued together, then added in ascending
      // slot order (an empty slot contributes 0 * 0)
      for (int j0 = 0; j0 < k; j0 += 8) {
        uint4 raw[8];
        float w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int j = j0 + u;
          const bool live = j < k && rows[j] >= 0;
          raw[u] = live ? __ldcs(reinterpret_cast<const uint4*>(y + (size_t)rows[j] * H + col)) : make_uint4(0u, 0u, 0u, 0u);
          w[u] = live ? wts[j] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          acc[0] = fmaf(w[u], cab::bf16_lo(raw[u].x), acc[0]); acc[1] = fmaf(w[u], cab::bf16_hi(raw[u].x), acc[1]);
          acc[2] = fmaf(w[u], cab::bf16_lo(raw[u].y), acc[2]); acc[3] = fmaf(w[u], cab::bf16_hi(raw[u].y), acc[3]);
          acc[4] = fmaf(w[u], cab::bf16_lo(raw[u].z), acc[4]); acc[5] = fmaf(w[u], cab::bf16_hi(raw[u].z), acc[5]);
          acc[6] = fmaf(w[u], cab::bf16_lo(raw[u].w), acc[6]); acc[7] = fmaf(w[u], cab::bf16_hi(raw[u].w), acc[7]);
        }
      }
      __nv_bfloat162 p0 = __floats2bfloat162_rn(acc[0], acc[1]), p1 = __floats2bfloat162_rn(acc[2], acc[3]);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[4], acc[5]), p3 = __floats2bfloat162_rn(acc[6], acc[7]);
      uint4 o;
      o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
      o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
      out[col >> 3] = o;
    }
  }
}

__global__ void fill_ones_kernel(float* p, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = 1.f;
}

Ctx* as_ctx(void* h) { return static_cast<Ctx*>(h); }

bool on_device(const Ctx* c) {
  int dev = -1;
  return cudaGetDevice(&dev) == cudaSuccess && dev == c->device;
}

}  // namespace

extern "C" size_t moe_ep_peer_buffer_bytes(int world, int t_cap, int H, int k) {
  if (world <= 0 || world > kMaxWorld || t_cap <= 0 || H <= 0 || H % 128 != 0 || k <= 0 || k > kMaxK) return 0;
  return make_layout(world, t_cap, H, k).bytes;
}

extern "C" int moe_ep_peer_create(void** ctx_out, int rank, int world, int t_cap, int H, int k, int e_local) {
  if (!ctx_out) return CAB_ERR_BAD_ARGUMENT;
  *ctx_out = nullptr;
  if (world <= 0 || world > kMaxWorld || rank < 0 || rank >= world || t_cap <= 0 || H <= 0 || H % 256 != 0 || k <= 0 ||
      k > kMaxK || e_local <= 0 || e_local > 256)
    return CAB_ERR_BAD_ARGUMENT;
  if ((long long)world * t_cap * k > (1LL << 30) || t_cap > 32768) return CAB_ERR_TOO_LARGE;
  Ctx* c = new (std::nothrow) Ctx();
  if (!c) return CAB_ERR_LAUNCH;
  c->L = make_layout(world, t_cap, H, k);
  c->rank = rank; c->e_local = e_local; c->epoch = 0; c->connected = false;
  for (int r = 0; r < kMaxWorld; ++r) { c->peers.base[r] = nullptr; c->ipc_opened[r] = false; }
  if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; return CAB_ERR_LAUNCH; }
  const size_t tw = (size_t)t_cap * world;
  const size_t local_bytes = tw * 4 * 2 + (size_t)world * 4 * 2 + tw * k * 4 + tw * 4 + 64;
  uint8_t* local = nullptr;
  if (cudaMalloc(&c->base, c->L.bytes) != cudaSuccess) { delete c; return CAB_ERR_LAUNCH; }
  if (cudaMalloc(&local, local_bytes) != cudaSuccess) { cudaFree(c->base); delete c; return CAB_ERR_LAUNCH; }
  // flags start at call number 0; everything else is written before it is read
  cudaMemset(c->base + c->L.off_flag, 0, kMaxWorld * 8);
  cudaMemset(c->base + c->L.off_back_flag, 0, kMaxWorld * 8);
  cudaMemset(local, 0, local_bytes);
  uint8_t* q = local;
  c->copy_pos = reinterpret_cast<int*>(q); q += tw * 4;
  c->back_row = reinterpret_cast<int*>(q); q += tw * 4;
  c->n_copies = reinterpret_cast<int*>(q); q += (size_t)world * 4;
  c->src_count = reinterpret_cast<int*>(q); q += (size_t)world * 4;
  c->keys = reinterpret_cast<int*>(q); q += tw * k * 4;
  c->ones = reinterpret_cast<float*>(q); q += tw * 4;
  q += 16;
  c->status = reinterpret_cast<int*>(q);
  fill_ones_kernel<<<(unsigned)((tw + 255) / 256), 256>>>(c->ones, tw);
  if (cudaDeviceSynchronize() != cudaSuccess) { cudaFree(c->base); cudaFree(local); delete c; return CAB_ERR_LAUNCH; }
  c->side_stream = nullptr; c->fork_event = nullptr; c->join_event = nullptr;
  if (cudaStreamCreateWithFlags(&c->side_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&c->fork_event, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&c->join_event, cudaEventDisableTiming) != cudaSuccess) {
    if (c->fork_event) cudaEventDestroy(c->fork_event);
    if (c->side_stream) cudaStreamDestroy(c->side_stream);
    cudaFree(c->base); cudaFree(local); delete c;
    cudaGetLastError();
    return CAB_ERR_LAUNCH;
  }
  c->peers.base[rank] = c->base;
  *ctx_out = c;
  return CAB_OK;
}

extern "C" int moe_ep_peer_export(void* ctx, void* handle64) {
  Ctx* c = as_ctx(ctx);
  if (!c || !handle64 || !on_device(c)) return CAB_ERR_BAD_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, c->base) != cudaSuccess) { cudaGetLastError(); return CAB_ERR_LAUNCH; }
  memcpy(handle64, &h, 64);
  return CAB_OK;
}

extern "C" int moe_ep_peer_connect_ipc(void* ctx, const void* handles) {
  Ctx* c = as_ctx(ctx);
  if (!c || !handles || !on_device(c) || c->connected) return CAB_ERR_BAD_ARGUMENT;
  for (int r = 0; r < c->L.world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)r * 64, 64);
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess || !p) {
      cudaGetLastError();
      return CAB_ERR_LAUNCH;
    }
    c->peers.base[r] = static_cast<uint8_t*>(p);
    c->ipc_opened[r] = true;
  }
  c->connected = true;
  return CAB_OK;
}

extern "C" int moe_ep_peer_connect_local(void* ctx, void* const* all_ctx) {
  Ctx* c = as_ctx(ctx);
  if (!c || !all_ctx || !on_device(c) || c->connected) return CAB_ERR_BAD_ARGUMENT;
  for (int r = 0; r < c->L.world; ++r) {
    const Ctx* o = as_ctx(all_ctx[r]);
    if (!o || o->rank != r || o->L.bytes != c->L.bytes) return CAB_ERR_BAD_ARGUMENT;
    if (o->device != c->device) {
      int can = 0;
      if (cudaDeviceCanAccessPeer(&can, c->device, o->device) != cudaSuccess || !can) return CAB_ERR_LAUNCH;
      const cudaError_t e = cudaDeviceEnablePeerAccess(o->device, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return CAB_ERR_LAUNCH; }
      cudaGetLastError();
    }
    c->peers.base[r] = o->base;
  }
  c->connected = true;
  return CAB_OK;
}

extern "C" int moe_ep_peer_destroy(void* ctx) {
  Ctx* c = as_ctx(ctx);
  if (!c) return CAB_OK;
  int caller_device = -1;
  cudaGetDevice(&caller_device);          // the caller's current device is put back before returning
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (int r = 0; r < kMaxWorld; ++r)
    if (c->ipc_opened[r]) cudaIpcCloseMemHandle(c->peers.base[r]);
  cudaEventDestroy(c->fork_event);
  cudaEventDestroy(c->join_event);
  cudaStreamDestroy(c->side_stream);
  cudaFree(c->copy_pos);     // first pointer of the local block
  cudaFree(c->base);
  delete c;
  if (caller_device >= 0) cudaSetDevice(caller_device);
  cudaGetLastError();
  return CAB_OK;
}

extern "C" int moe_ep_peer_debug_read(void* ctx, int which, size_t offset, void* dst, size_t bytes) {
  Ctx* c = as_ctx(ctx);
  if (!c || !dst || !on_device(c)) return CAB_ERR_BAD_ARGUMENT;
  const Layout& L = c->L;
  const size_t tw = (size_t)L.t_cap * L.world;
  const uint8_t* src = nullptr;
  size_t extent = 0;
  switch (which) {
    case 0: src = c->base + L.off_rows; extent = tw * L.H; break;
    case 1: src = c->base + L.off_side; extent = tw * L.side_ld * 4; break;
    case 2: src = c->base + L.off_back; extent = tw * L.H * 2; break;
    case 3: src = reinterpret_cast<const uint8_t*>(c->keys); extent = tw * L.k * 4; break;
    case 4: src = reinterpret_cast<const uint8_t*>(c->src_count); extent = (size_t)L.world * 4; break;
    case 5: src = reinterpret_cast<const uint8_t*>(c->copy_pos); extent = tw * 4; break;
    default: return CAB_ERR_BAD_ARGUMENT;
  }
  if (offset > extent || bytes > extent - offset) return CAB_ERR_BAD_ARGUMENT;
  return cudaMemcpy(dst, src + offset, bytes, cudaMemcpyDefault) == cudaSuccess ? CAB_OK : CAB_ERR_LAUNCH;
}

extern "C" int moe_ep_peer_dispatch_launcher(void* ctx, const cab_bf16* x, const int* topk_idx, const float* topk_w,
                                             int T, int config, cudaStream_t stream) {
  (void)config;
  Ctx* c = as_ctx(ctx);
  if (!c || !c->connected || !on_device(c)) return CAB_ERR_BAD_ARGUMENT;
  if (T < 0 || T > c->L.t_cap || (T > 0 && (!x || !topk_idx || !topk_w))) return CAB_ERR_BAD_ARGUMENT;
  if (T > 0 && !cab::aligned_to(x, 16)) return CAB_ERR_MISALIGNED;
  const Layout& L = c->L;
  c->epoch += 1;                       // this call's number; every rank makes the same sequence of calls
  ep_plan_kernel<<<L.world, 1024, 0, stream>>>(topk_idx, T, L.k, c->e_local, L.world, L.t_cap, c->copy_pos,
                                               c->back_row, c->n_copies);
  const long long warps = (long long)T * ((L.H + 1023) >> 10);
  const unsigned grid = warps > 0 ? (unsigned)((warps + 7) / 8) : 1u;
  ep_dispatch_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), topk_idx, topk_w,
                                               c->copy_pos, T, c->rank, c->e_local, L, c->peers);
  ep_publish_kernel<<<1, 32, 0, stream>>>(c->peers, L.off_flag, c->rank, L.world, c->epoch, c->n_copies);
  return cab::launch_status();
}

extern "C" int moe_ep_peer_receive_launcher(void* ctx, int config, cudaStream_t stream) {
  (void)config;
  Ctx* c = as_ctx(ctx);
  if (!c || !c->connected || !on_device(c) || c->epoch == 0) return CAB_ERR_BAD_ARGUMENT;
  const Layout& L = c->L;
  ep_wait_flags_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const unsigned long long*>(c->base + L.off_flag), L.world,
                                             c->epoch, L.t_cap, c->src_count, c->status + 0, kWaitDispatch);
  const long long total = (long long)L.world * L.t_cap * L.k;
  ep_keys_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const uint32_t*>(c->base + L.off_side), c->src_count, L.world, L.t_cap, L.k, L.side_ld, L.nb,
      c->e_local, c->keys);
  return cab::launch_status();
}

extern "C" int moe_ep_peer_gather_launcher(void* ctx, cab_e4m3* a_q, float* a_scales_t, const int* dst_row,
                                           int ld_rows, int config, cudaStream_t stream) {
  (void)config;
  Ctx* c = as_ctx(ctx);
  if (!c || !c->connected || !on_device(c) || !a_q || !a_scales_t || !dst_row || ld_rows <= 0)
    return CAB_ERR_BAD_ARGUMENT;
  if (!cab::aligned_to(a_q, 16)) return CAB_ERR_MISALIGNED;
  const Layout& L = c->L;
  ep_gather_kernel<<<cab::kNumSMs * 4, cab::row_walk_threads(L.H / 16), 0, stream>>>(a_q, a_scales_t, c->base + L.off_rows,
                                                         reinterpret_cast<const float*>(c->base + L.off_side),
                                                         c->src_count, dst_row, L.world, L.t_cap, L.k, L.H, L.side_ld,
                                                         ld_rows);
  return cab::launch_status();
}

extern "C" int moe_ep_peer_return_launcher(void* ctx, const cab_bf16* y, const int* dst_row, int config,
                                           cudaStream_t stream) {
  Ctx* c = as_ctx(ctx);
  if (!c || !c->connected || !on_device(c) || !y || !dst_row) return CAB_ERR_BAD_ARGUMENT;
  if (!cab::aligned_to(y, 16)) return CAB_ERR_MISALIGNED;
  const Layout& L = c->L;
  const int grid = config > 0 ? config : cab::kNumSMs * 4;
  ep_return_kernel<<<grid, cab::row_walk_threads(L.H / 8), 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(y),
                                             reinterpret_cast<const float*>(c->base + L.off_side), c->src_count,
                                             dst_row, c->rank, L, c->peers);
  ep_publish_kernel<<<1, 32, 0, stream>>>(c->peers, L.off_back_flag, c->rank, L.world, c->epoch, nullptr);
  return cab::launch_status();
}

extern "C" int moe_ep_peer_combine_launcher(void* ctx, cab_bf16* out, const cab_bf16* shared, int T, int config,
                                            cudaStream_t stream) {
  Ctx* c = as_ctx(ctx);
  if (!c || !c->connected || !on_device(c) || T < 0 || T > c->L.t_cap || (T > 0 && !out)) return CAB_ERR_BAD_ARGUMENT;
  const Layout& L = c->L;
  ep_wait_flags_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const unsigned long long*>(c->base + L.off_back_flag),
                                             L.world, c->epoch, L.t_cap, nullptr, c->status + 1, kWaitReturn);
  if (cab::launch_status() != CAB_OK) return CAB_ERR_LAUNCH;
  return moe_combine_launcher(out, reinterpret_cast<const cab_bf16*>(c->base + L.off_back), c->back_row, c->ones, shared,
                              T, L.H, L.world, config, stream);
}

// ------------------------------------------------------------------ the whole layer
namespace {

struct Workspace {
  float* logits; int* idx; float* w;
  int *counts, *offsets, *pad_offsets, *perm, *inv_perm, *dst_row, *tile_expert, *num_tiles, *status;
  void* permute_scratch;
  uint8_t* a_q; float* a_s; uint8_t* h_q; float* h_s; uint8_t* y;
  uint8_t* xs_q; float* xs_s; uint8_t* hs_q; float* hs_s; uint8_t* y_shared;
  int max_tiles, cap, shared_tiles, scap;
  size_t bytes;
};

// Carves the workspace; with base == nullptr only the size is computed.
Workspace carve(const Ctx* c, const cab_moe_ep_layer_args* a, uint8_t* base) {
  const Layout& L = c->L;
  Workspace w;
  size_t o = 0;
  auto take = [&](size_t bytes) { uint8_t* p = base ? base + o : nullptr; o = (o + bytes + 255) & ~size_t(255); return p; };
  const size_t t = L.t_cap, n = (size_t)L.world * L.t_cap * L.k;
  w.max_tiles = (a->entry_cap + 127) / 128 + c->e_local;
  w.cap = w.max_tiles * 128;
  w.shared_tiles = (L.t_cap + 127) / 128;
  w.scap = w.shared_tiles * 128;
  const size_t H = L.H, I = a->I, nb = L.nb;
  w.logits = (float*)take(t * a->E * 4);
  w.idx = (int*)take(t * L.k * 4);
  w.w = (float*)take(t * L.k * 4);
  w.counts = (int*)take((size_t)(c->e_local + 1) * 4);
  w.offsets = (int*)take((size_t)(c->e_local + 1) * 4);
  w.pad_offsets = (int*)take((size_t)(c->e_local + 1) * 4);
  w.perm = (int*)take(n * 4);
  w.inv_perm = (int*)take(n * 4);
  w.dst_row = (int*)take(n * 4);
  w.tile_expert = (int*)take((size_t)w.max_tiles * 4);
  w.num_tiles = (int*)take(4);
  w.status = (int*)take(8 * 4);
  w.permute_scratch = take(moe_permute_scratch_bytes(L.world * L.t_cap, L.k, c->e_local));
  w.a_q = take((size_t)w.cap * H);
  w.a_s = (float*)take(nb * w.cap * 4);
  w.h_q = take((size_t)w.cap * I);
  w.h_s = (float*)take((I / 128) * (size_t)w.cap * 4);
  w.y = take((size_t)w.cap * H * 2);
  const bool sh = a->shared_w13_q != nullptr;
  w.xs_q = take(sh ? (size_t)w.scap * H : 0);
  w.xs_s = (float*)take(sh ? nb * w.scap * 4 : 0);
  w.hs_q = take(sh ? (size_t)w.scap * I : 0);
  w.hs_s = (float*)take(sh ? (I / 128) * (size_t)w.scap * 4 : 0);
  w.y_shared = take(sh ? (size_t)w.scap * H * 2 : 0);
  w.bytes = o;
  return w;
}

bool layer_args_ok(const Ctx* c, const cab_moe_ep_layer_args* a) {
  if (!c || !a) return false;
  if (!a->router_w || !a->w13_q || !a->w13_s || !a->w2_q || !a->w2_s) return false;
  if (a->E != c->e_local * c->L.world || a->I <= 0 || a->I % 128 != 0 || a->entry_cap <= 0) return false;
  if (a->routing != 0 && a->routing != 1) return false;
  if (a->routing == 1 && !a->router_bias) return false;
  const bool any = a->shared_w13_q || a->shared_w13_s || a->shared_w2_q || a->shared_w2_s;
  const bool all = a->shared_w13_q && a->shared_w13_s && a->shared_w2_q && a->shared_w2_s;
  return any == all;
}

}  // namespace

extern "C" size_t moe_ep_peer_workspace_bytes(void* ctx, const cab_moe_ep_layer_args* args) {
  const Ctx* c = as_ctx(ctx);
  if (!layer_args_ok(c, args)) return 0;
  return carve(c, args, nullptr).bytes;
}

#define EP_TRY(expr)                   \
  do {                                 \
    const int rc_ = (expr);            \
    if (rc_ != CAB_OK) return rc_;     \
  } while (0)

extern "C" int moe_ep_peer_layer_launcher(void* ctx, cab_bf16* out, const cab_bf16* x, int T,
                                          const cab_moe_ep_layer_args* a, void* workspace, size_t workspace_bytes,
                                          int config, cudaStream_t stream) {
  Ctx* c = as_ctx(ctx);
  if (!layer_args_ok(c, a) || !c->connected || !on_device(c) || !workspace) return CAB_ERR_BAD_ARGUMENT;
  if (T < 0 || T > c->L.t_cap || (T > 0 && (!out || !x))) return CAB_ERR_BAD_ARGUMENT;
  if (!cab::aligned_to(workspace, 256)) return CAB_ERR_MISALIGNED;
  const Workspace w = carve(c, a, static_cast<uint8_t*>(workspace));
  if (workspace_bytes < w.bytes) return CAB_ERR_BAD_ARGUMENT;
  const Layout& L = c->L;
  const int H = L.H, I = a->I, k = L.k;
  const bool has_shared = a->shared_w13_q != nullptr;

  // config selects stages (bit 0: routing, dispatch and the shared expert; bit 1: receive, GEMMs, return;
  // bit 2: combine); 0 runs all of them. Ranks that share one GPU are stepped stage by stage, so that no
  // launch ever waits for a flag that a later launch on the same GPU would publish.
  const int stages = (config & 7) ? (config & 7) : 7;

  if (stages & 1) {
    // the four GEMM status words start at zero (a launch that runs clears its own; the shared expert's
    // two stay untouched when there is none)
    if (cudaMemsetAsync(w.status, 0, 8 * sizeof(int), stream) != cudaSuccess) return CAB_ERR_LAUNCH;
    // routing of the local tokens
    EP_TRY(moe_router_logits_launcher(w.logits, x, a->router_w, T, H, a->E, 0, stream));
    if (a->routing == 0)
      EP_TRY(moe_route_softmax_topk_launcher(w.idx, w.w, w.logits, T, a->E, k, 0, stream));
    else
      EP_TRY(moe_route_sigmoid_group_topk_launcher(w.idx, w.w, w.logits, a->router_bias, T, a->E, k, a->n_group,
                                                   a->topk_group, a->scaling, 0, stream));
    // the shared expert needs nothing that is exchanged: it runs on the side stream from here on
    if (has_shared && T > 0) {
      if (cudaEventRecord(c->fork_event, stream) != cudaSuccess ||
          cudaStreamWaitEvent(c->side_stream, c->fork_event, 0) != cudaSuccess)
        return CAB_ERR_LAUNCH;
    }
    EP_TRY(moe_ep_peer_dispatch_launcher(ctx, x, w.idx, w.w, T, 0, stream));
    if (has_shared && T > 0) {
      cudaStream_t ss = c->side_stream;
      EP_TRY(moe_quant_dispatch_launcher(w.xs_q, w.xs_s, x, nullptr, T, H, 1, w.scap, 0, ss));
      const int tiles = (T + 127) / 128;
      EP_TRY(moe_grouped_gemm_fp8_launcher(0, w.hs_q, w.hs_s, w.xs_q, w.xs_s, a->shared_w13_q, a->shared_w13_s,
                                           nullptr, nullptr, tiles, w.scap, w.scap, 1, I, H, w.status + 2,
                                           a->gemm_ctas, ss));
      EP_TRY(moe_grouped_gemm_fp8_launcher(1, w.y_shared, nullptr, w.hs_q, w.hs_s, a->shared_w2_q, a->shared_w2_s,
                                           nullptr, nullptr, tiles, w.scap, w.scap, 1, H, I, w.status + 3,
                                           a->gemm_ctas, ss));
      if (cudaEventRecord(c->join_event, ss) != cudaSuccess) return CAB_ERR_LAUNCH;
    }
  }
  if (stages & 2) {
    // arrivals -> padded row space of the local experts -> grouped GEMMs -> partial results back
    EP_TRY(moe_ep_peer_receive_launcher(ctx, 0, stream));
    EP_TRY(moe_permute_launcher(c->keys, L.world * L.t_cap, k, c->e_local, w.counts, w.offsets, w.pad_offsets,
                                w.perm, w.inv_perm, w.dst_row, w.tile_expert, w.num_tiles, w.max_tiles,
                                w.permute_scratch, 1 /* -1 marks an empty slot */, stream));
    EP_TRY(moe_ep_peer_gather_launcher(ctx, w.a_q, w.a_s, w.dst_row, w.cap, 0, stream));
    EP_TRY(moe_grouped_gemm_fp8_launcher(0, w.h_q, w.h_s, w.a_q, w.a_s, a->w13_q, a->w13_s, w.tile_expert,
                                         w.num_tiles, w.max_tiles, w.cap, w.cap, c->e_local, I, H, w.status + 0,
                                         a->gemm_ctas, stream));
    EP_TRY(moe_grouped_gemm_fp8_launcher(1, w.y, nullptr, w.h_q, w.h_s, a->w2_q, a->w2_s, w.tile_expert, w.num_tiles,
                                         w.max_tiles, w.cap, w.cap, c->e_local, H, I, w.status + 1, a->gemm_ctas,
                                         stream));
    EP_TRY(moe_ep_peer_return_launcher(ctx, reinterpret_cast<const cab_bf16*>(w.y), w.dst_row, 0, stream));
  }
  if (stages & 4) {
    if (has_shared && T > 0 && cudaStreamWaitEvent(stream, c->join_event, 0) != cudaSuccess) return CAB_ERR_LAUNCH;
    EP_TRY(moe_ep_peer_combine_launcher(
        ctx, out, has_shared && T > 0 ? reinterpret_cast<const cab_bf16*>(w.y_shared) : nullptr, T, 0, stream));
  }
  return CAB_OK;
}

// Blocking read of the layer's status words: [0..3] the four GEMM launches' give-up codes (routed gate/up,
// routed down, shared gate/up, shared down), [4] the permutation flag (1 = bad expert id, 2 = more entries
// than entry_cap holds), [5] wait for dispatch flags (301 = ran out), [6] wait for return flags (302).
extern "C" int moe_ep_peer_read_status(void* ctx, const cab_moe_ep_layer_args* a, void* workspace, int* host_out8) {
  Ctx* c = as_ctx(ctx);
  if (!layer_args_ok(c, a) || !workspace || !host_out8 || !on_device(c)) return CAB_ERR_BAD_ARGUMENT;
  const Workspace w = carve(c, a, static_cast<uint8_t*>(workspace));
  int gemm[4], flag = 0, waits[4];
  const int* permute_flag = reinterpret_cast<const int*>(w.permute_scratch) +
                            moe_permute_scratch_bytes(c->L.world * c->L.t_cap, c->L.k, c->e_local) / 4 - 1;
  if (cudaMemcpy(gemm, w.status, sizeof(gemm), cudaMemcpyDeviceToHost) != cudaSuccess ||
      cudaMemcpy(&flag, permute_flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess ||
      cudaMemcpy(waits, c->status, sizeof(waits), cudaMemcpyDeviceToHost) != cudaSuccess)
    return CAB_ERR_LAUNCH;
  for (int i = 0; i < 4; ++i) host_out8[i] = gemm[i];
  host_out8[4] = flag; host_out8[5] = waits[0]; host_out8[6] = waits[1]; host_out8[7] = 0;
  return CAB_OK;
}
