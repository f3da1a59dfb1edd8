/* CPU oracle for the MTP speculative-decode path -- TEST INFRASTRUCTURE ONLY.
 *
 * A scalar restatement of the reference's algorithms for this path. It is the checker for the
 * CUDA kernels: only the test suite, the smoke check and the CPU-baseline leg of the benchmark
 * may load it. The product library never links, loads or calls anything declared here.
 *
 * Parity status: the Q4_K dequantisation and the f16 conversions are pinned against the
 * reference's own host code (engine/src/quant.h, compiled into oracle/_ref by the Makefile);
 * the GEMV is pinned through the reference's own acceptance rule (engine/bench/bench_gemv.cpp:96-111:
 * |ref - got| / sum|w*x| < 1e-5 against dequant_row(...) . x accumulated in double).
 * The kernels that exist in the reference only as HIP device code (norms, GDN, attention, router,
 * argmax) have no host twin and no checked-in golden vectors there: for those the restatement
 * follows the device source line by line and parity is pinned only by the reference's own
 * property tests (sequential-vs-batched GDN, spec stream == plain stream): "parity unpinned"
 * beyond those properties.
 *
 * Every function cites the reference file:line it follows (paths relative to the reference root).
 */
#pragma once
#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- formats (engine/src/quant.h:11-17,22,37-53,150-155) ---- */
float    orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float f);
/* 8 (scale, min) 6-bit pairs of one Q4_K block: quant.h:37-40 */
void orc_q4k_scale_min(const uint8_t scales[12], uint8_t sc[8], uint8_t mn[8]);
/* dequantise nblk consecutive 144-byte Q4_K blocks to 256*nblk floats: quant.h:43-53 */
void orc_dequant_q4k(const uint8_t* blocks, size_t nblk, float* y);

/* ---- deterministic transcendental functions shared by definition with the device code ---- */
float orc_expf(float x);
float orc_log1pf_pos(float e);  /* log(1+e) for e >= 0 */
float orc_sigmoid(float x);     /* ops.hip:12 */
float orc_silu(float x);        /* ops.hip:11 */
float orc_softplus(float x);    /* ops.hip:13 */

/* ---- activation quantiser: engine/kernels/gemv.hip:36-51 == engine/bench/bench_gemv.cpp:17-25 ---- */
/* x [R][K] f32 -> q [R][K] i8, d [R][K/32], s [R][K/32] */
void orc_quantize_x_q8(const float* x, int R, int K, int8_t* q, float* d, float* s);

/* ---- Q4_K GEMV ---- */
/* f32 activations, arithmetic and lane partition of k_gemv_q4_K_f32 (gemv.hip:1177-1216) with TPR lanes/row.
 * y [R][N]. */
void orc_gemv_q4k_f32(const uint8_t* W, const float* x, float* y, int N, int K, int R, int tpr);
/* W4A8: exact int32 dot per 32-element sub-block, one fp32 update per sub-block in block order
 * (gemv.hip:602-672 numerics contract); split-K partial sums are added in a fixed, shape-only order (see the .cpp).
 * y [R][ldy] (row stride ldy >= N). */
void orc_gemv_q4k_q8(const uint8_t* W, const int8_t* q, const float* d, const float* s, float* y, int N, int K, int R, int ldy);
/* reference check of bench_gemv.cpp:97-104: dequantised row . x in double; also returns sum|w*x| */
void orc_gemv_q4k_double(const uint8_t* W, const float* x, double* y, double* mag, int N, int K, int R);

/* ---- argmax + greedy acceptance: ops.hip:702-716 (max value, lowest index), spec27b.cpp:92-97 ---- */
void orc_argmax(const float* logits, int R, int n, int ld, int* ids, float* vals);
/* top-k per row (ops.hip:702-716): ids / vals [R][k], values descending, ties -> lower index */
void orc_topk(const float* logits, int R, int n, int ld, int k, int* ids, float* vals);
/* ids [n_draft+1] = target argmax per verify row; returns mm = accepted drafts; *bonus = ids[mm] */
int orc_accept(const int* ids, const int* drafts, int n_draft, int* bonus);

int orc_num_threads(void);

#ifdef __cplusplus
}
#endif
