// Internal C++ launchers of the CUDA kernels (device pointers + stream), the layer the reference calls
// "kernels" (engine/kernels/gemv.h, ops.h, fn.h). The C ABI in capi.cu and the engine sit on top of these.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

namespace hp {

// Quantised activations in the fragment-major layout described in hp_common.cuh (reference: struct XQ8, gemv.h:8).
struct XQ8F { void* q; void* sc; };

// device status word (set by kernels whose bounded waits gave up); nullptr if it cannot be allocated
int* device_err_flag();

// ---- gemv_q4k.cu ----
int gemv_q4k_q8(const void* W, const XQ8F& x, float* y, int N, int K, int R, int ldy, int* err, cudaStream_t s, bool pdl);
int gemv_q4k_f32(const void* W, const float* x, float* y, int N, int K, int R, cudaStream_t s);

// ---- quant_ops.cu ----
int quantize_x_q8(const float* x, int ldx, XQ8F out, int R, int K, cudaStream_t s);
int xq8_unpack(XQ8F in, int R, int K, int8_t* q, float* d, float* sm, cudaStream_t s);
int dequant_q4k(const void* W, size_t nblk, float* out, cudaStream_t s);

// ---- argmax.cu ----
// per-row argmax (max value, lowest index) of logits [R][ld] -> ids/vals on device
int argmax_rows(const float* logits, int R, int n, int ld, int* ids, float* vals, void* scratch, cudaStream_t s);
size_t argmax_scratch_bytes(int R, int n);
// greedy prefix acceptance on device: out[0] = accepted drafts mm, out[1] = bonus id ids[mm]
int accept_greedy(const int* ids, const int* drafts, int n_draft, int* out, cudaStream_t s);

}  // namespace hp
