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

// AdamW (decoupled weight decay, bias correction as torch.optim.AdamW) over a list of tensors: one launch per 80
// tensors plus one for the step counter.  `tensors` is a HOST array; it travels in the kernels' parameter space, so
// nothing is uploaded or allocated and the call can be captured in a CUDA graph.  paramType is the storage type of
// parameters and gradients, stateType that of the two moments: bf16/bf16, fp32/fp32, or bf16 parameters with fp32
// moments; tensors whose four pointers are not 16-byte aligned run element by element.  stepState: 4 floats in device memory owned by the caller,
// [0] = steps taken so far (start at 0; the call increments it on the device), [1..2] scratch for the bias corrections.
// lrDev != NULL: the learning rate is read from device memory at run time (schedulers under graph replay), else `lr`.
typedef struct {
    void* param;
    const void* grad;
    void* expAvg;
    void* expAvgSq;
    uint64_t numel;
} HcclAdamTensor;
HcclResult HcclFusedAdamW(const HcclAdamTensor* tensors, uint32_t nTensors, HcclDataType paramType, HcclDataType stateType, float lr,
                          const float* lrDev, float beta1, float beta2, float eps, float weightDecay, float* stepState, hcclStream_t stream);
// Kernel launches a call with nTensors tensors makes.
uint32_t HcclFusedAdamWLaunches(uint32_t nTensors);

#ifdef __cplusplus
}
#endif
#endif
