// Single-pass bf16 kernels for the memory-bound pieces of a decoder layer (residual add + RMSNorm, SwiGLU, rotary
// embedding), forward and backward.  No counterpart in the reference (a communication library): they serve the
// tensor-parallel decoder stack the fused matmul + collective kernels are measured in.  All tensors are bf16 and
// 16-byte aligned unless stated; math is fp32.  Nothing is allocated; work is enqueued on `stream`.
#ifndef HCCL_FUSED_OPS_H
#define HCCL_FUSED_OPS_H
#include "hccl_types.h"
#ifdef __cplusplus
extern "C" {
#endif

// xOut = x + delta (skipped when delta == NULL; xOut may then be NULL), h = xOut * rstd * w with
// rstd[row] = rsqrt(mean(xOut[row]^2) + eps) stored as fp32.  hidden: multiple of 8, at most 8192.
HcclResult HcclFusedAddRmsNormFwd(const void* x, const void* delta, const void* w, void* xOut, void* h, void* rstd, uint64_t rows, uint32_t hidden,
                                  float eps, hcclStream_t stream);
// Number of fp32 partial rows HcclFusedRmsNormBwd needs in dwPartial ([partials][hidden]).
uint32_t HcclFusedRmsNormBwdPartials(uint64_t rows);
// dx = rstd * (dh * w) - x * rstd^3 * mean(dh * w * x) (+ dxExtra when not NULL), dw = sum_rows dh * x * rstd.
HcclResult HcclFusedRmsNormBwd(const void* dh, const void* x, const void* w, const void* rstd, const void* dxExtra, void* dx, void* dwPartial,
                               void* dw, uint64_t rows, uint32_t hidden, hcclStream_t stream);
// gu [rows, 2f] = [gate | up]: out [rows, f] = silu(gate) * up; backward writes dgu [rows, 2f].  f: multiple of 8.
HcclResult HcclFusedSwigluFwd(const void* gu, void* out, uint64_t rows, uint32_t f, hcclStream_t stream);
HcclResult HcclFusedSwigluBwd(const void* gu, const void* dout, void* dgu, uint64_t rows, uint32_t f, hcclStream_t stream);
// Rotary embedding ("rotate halves") of nHeads heads of headDim (multiple of 16) per row; rows of in / out are
// inStride / outStride elements apart (multiples of 8); cos / sin: fp32 [rows, headDim / 2].  backward != 0 applies
// the transposed rotation (for gradients).
HcclResult HcclFusedRope(const void* in, uint64_t inStride, void* out, uint64_t outStride, const void* cosTable, const void* sinTable, uint64_t rows,
                         uint32_t nHeads, uint32_t headDim, int backward, hcclStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
