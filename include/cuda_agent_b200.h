/*
 * C ABI of libcuda_agent_b200.so: the kernel launchers of the B200 (sm_100a)
 * operators that sit behind the agent_workdir binding API.
 *
 * Convention (reference: agent_workdir/kernels/axpby.cu:12-20 and the extern
 * declaration a binding file repeats, agent_workdir/kernels/axpby_binding.cpp:7-15):
 *   extern "C" <op>_launcher(raw device pointers, sizes, scalars, int config,
 *                            cudaStream_t stream)
 * - every pointer is a device pointer owned by the caller; nothing is copied,
 *   nothing is allocated unless a launcher's comment says so;
 * - work is enqueued on `stream` and the call returns without synchronising;
 * - `config` selects a launch variant of the same arithmetic (tuning knob,
 *   agent_workdir/kernels/axpby.cu:22-41); every value gives identical results
 *   unless stated otherwise; unknown values fall back to the default variant.
 * The reference launcher returns void and checks nothing. These return an int
 * status (CAB_OK == 0) so that a binding can raise; a caller that ignores the
 * return value sees the reference behaviour.
 *
 * No torch type appears here. `cudaStream_t` is spelled as an opaque pointer so
 * the header is usable from plain C and from ctypes/cffi.
 */
#ifndef CUDA_AGENT_B200_H_
#define CUDA_AGENT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same type that cuda_runtime.h names cudaStream_t (driver_types.h:
 * `typedef struct CUstream_st* cudaStream_t`), spelled out so that this header
 * needs no CUDA header. */
typedef struct CUstream_st* cab_stream_t;

/* 16-bit storage types: raw IEEE bfloat16 bits / e4m3 bytes. */
typedef uint16_t cab_bf16;
typedef uint8_t cab_e4m3;

enum cab_status {
  CAB_OK = 0,
  CAB_ERR_BAD_ARGUMENT = 1,   /* null pointer, non-positive size, unsupported head size ... */
  CAB_ERR_MISALIGNED = 2,     /* a pointer that must be 16-byte aligned is not */
  CAB_ERR_LAUNCH = 3,         /* cudaGetLastError() was non-zero after the launch */
  CAB_ERR_TOO_LARGE = 4,      /* a size exceeds what the entry point supports */
  CAB_ERR_DEVICE_STATUS = 5   /* a kernel's own bounded wait or index check gave up */
};

/* Human-readable text for a status code (static storage). */
const char* cab_status_string(int status);

/* Library version as major*10000 + minor*100 + patch. */
int cab_version(void);

/* ------------------------------------------------------------------------- */
/* axpby: the workspace's smoke-test op.                                      */
/* Replaces agent_workdir/kernels/axpby.cu:12-42 (same argument order).       */
/* out[i] = alpha * a[i] + b[i], fp32. config: 0 -> 256, 1 -> 128, 2 -> 512    */
/* threads per block. size <= 0 is a no-op returning CAB_OK.                  */
/* ------------------------------------------------------------------------- */
int axpby_launcher(float* out, const float* a, const float* b, float alpha, int size, int config,
                   cab_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Gated DeltaNet single-step decode.                                         */
/* The reference ships no such op; this fills the slot an op occupies in       */
/* agent_workdir/kernels/ (launcher ABI as above) for the eager statement      */
/*   alpha = exp(g);  u = S k;  S' = alpha*S + beta*(v - alpha*u) k^T;          */
/*   o = S' q / sqrt(128)                                                      */
/* per (batch b, value head hv), which equals                                  */
/*   S' = alpha * S (I - beta k k^T) + beta v k^T.                             */
/*                                                                             */
/* state : fp32 [B, Hv, 128 (dv), 128 (dk)] row-major, UPDATED IN PLACE        */
/* out   : fp32 [B, Hv, 128]                                                   */
/* q, k  : bf16 [B, Hq, 128]  (value head hv reads q/k head hv / (Hv/Hq))      */
/* v     : bf16 [B, Hv, 128]                                                   */
/* g     : fp32 [B, Hv]  log-decay (<= 0);   beta : fp32 [B, Hv]               */
/* Requires Hv % Hq == 0; state and out 16-byte aligned, q/k/v 8-byte aligned. */
/* config: 0 default (8 rows in flight per warp), 1 -> 4 rows, 2 -> 16 rows.    */
/* One launch reads and writes each state element exactly once.               */
/* ------------------------------------------------------------------------- */
int gdn_decode_launcher(float* state, float* out, const cab_bf16* q, const cab_bf16* k,
                        const cab_bf16* v, const float* g, const float* beta, int B, int Hq,
                        int Hv, int config, cab_stream_t stream);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* CUDA_AGENT_B200_H_ */
