// Activation quantiser and Q4_K dequantisation kernels.
// Reference: k_quantize_x_q8 (engine/kernels/gemv.hip:36-51), dequant_q4_K (engine/src/quant.h:43-53),
// k_embed_q4_K (engine/kernels/ops.hip:154-171).
#include "hp_common.cuh"
#include "kernels.h"

namespace hp {
namespace {

// warp per 32-element sub-block; grid (ceil(K/32/8), R)
__global__ void __launch_bounds__(256) k_quantize_x_q8(const float* __restrict__ x, int ldx, int8_t* __restrict__ q, float* __restrict__ sc, int K) {
    const int r = blockIdx.y, sb = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (sb * 32 >= K) return;
    warp_quant32_store(x[(size_t)r * ldx + sb * 32 + lane], r, sb, K, q, sc, lane);
}

__global__ void k_xq8_unpack(const int8_t* __restrict__ q, const float* __restrict__ sc, int R, int K, int8_t* __restrict__ oq, float* __restrict__ od, float* __restrict__ os) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * K) return;
    const int r = (int)(i / K), k = (int)(i % K);
    oq[i] = q[xq_q_index(r, k, K)];
    if ((k & 31) == 0) { const size_t di = xq_d_index(r, k >> 5, K); od[(size_t)r * (K / 32) + (k >> 5)] = sc[di]; os[(size_t)r * (K / 32) + (k >> 5)] = sc[di + 2]; }
}

// thread per element: block b, element e = 64g + 32h + l -> nibble h of byte 32g + l, (scale, min) 2g + h
__global__ void __launch_bounds__(256) k_dequant_q4k(const uint8_t* __restrict__ W, size_t nblk, float* __restrict__ out) {
    const size_t b = blockIdx.x; if (b >= nblk) return;
    const uint8_t* blk = W + b * 144;
    const int e = threadIdx.x, g = e >> 6, h = (e >> 5) & 1, l = e & 31;
    const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));
    const float d = h2f((uint16_t)(hdr.x & 0xFFFF)), dmin = h2f((uint16_t)(hdr.x >> 16));
    uint32_t sc, mn; q4k_scale_min(hdr, 2 * g + h, sc, mn);
    const uint32_t qb = blk[16 + 32 * g + l];
    const float qv = (float)(h ? (qb >> 4) : (qb & 0xFu));
    out[b * 256 + e] = (d * (float)sc) * qv - dmin * (float)mn;
}

}  // namespace

int quantize_x_q8(const float* x, int ldx, XQ8F out, int R, int K, cudaStream_t s) {
    HP_REQUIRE(K > 0 && K % 64 == 0 && R >= 1 && ldx >= K, "quantize_x_q8: bad shape R=%d K=%d ldx=%d", R, K, ldx);
    dim3 grid((K / 32 + 7) / 8, R);
    k_quantize_x_q8<<<grid, 256, 0, s>>>(x, ldx, (int8_t*)out.q, (float*)out.sc, K);
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}
int xq8_unpack(XQ8F in, int R, int K, int8_t* q, float* d, float* sm, cudaStream_t s) {
    const size_t n = (size_t)R * K;
    k_xq8_unpack<<<(unsigned)((n + 255) / 256), 256, 0, s>>>((const int8_t*)in.q, (const float*)in.sc, R, K, q, d, sm);
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}
int dequant_q4k(const void* W, size_t nblk, float* out, cudaStream_t s) {
    HP_REQUIRE(nblk > 0 && nblk < (1ull << 31), "dequant_q4k: bad block count");
    k_dequant_q4k<<<(unsigned)nblk, 256, 0, s>>>((const uint8_t*)W, nblk, out);
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}

}  // namespace hp
