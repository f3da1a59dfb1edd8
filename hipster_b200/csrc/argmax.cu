// Per-row argmax over the vocabulary and greedy prefix acceptance, on device.
// Reference: k_topk with k = 1 (engine/kernels/ops.hip:702-716: maximum value, ties -> lowest index) and the
// host acceptance loop of the MTP driver (engine/bench/spec27b.cpp:92-97). The reference copies the ids to the
// host and compares there; here the comparison runs on the device so that no logits or ids round-trip is needed.
#include "hp_common.cuh"
#include "kernels.h"

namespace hp {
namespace {

constexpr int AM_CHUNK = 8192;   // elements per stage-1 block

__device__ __forceinline__ void am_better(float& bv, int& bi, float v, int i) {
    if (v > bv || (v == bv && i < bi && i >= 0)) { bv = v; bi = i; }
}
__device__ __forceinline__ void am_block_reduce(float& bv, int& bi, float* sv, int* si) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off); const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        am_better(bv, bi, ov, oi);
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) { sv[w] = bv; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
        bv = l < (int)(blockDim.x >> 5) ? sv[l] : -INFINITY; bi = l < (int)(blockDim.x >> 5) ? si[l] : -1;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off); const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            am_better(bv, bi, ov, oi);
        }
    }
}
__global__ void __launch_bounds__(256) k_argmax_part(const float* __restrict__ x, int n, int ld, float* __restrict__ pv, int* __restrict__ pi) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sv[8]; __shared__ int si[8];
    const int r = blockIdx.y, c0 = blockIdx.x * AM_CHUNK, c1 = min(n, c0 + AM_CHUNK);
    const float* xr = x + (size_t)r * ld;
    float bv = -INFINITY; int bi = -1;
    for (int i = c0 + threadIdx.x; i < c1; i += 256) { const float v = xr[i]; if (v > bv) { bv = v; bi = i; } }
    am_block_reduce(bv, bi, sv, si);
    if (threadIdx.x == 0) { pv[(size_t)r * gridDim.x + blockIdx.x] = bv; pi[(size_t)r * gridDim.x + blockIdx.x] = bi; }
}
__global__ void __launch_bounds__(256) k_argmax_final(const float* __restrict__ pv, const int* __restrict__ pi, int np, int* __restrict__ ids, float* __restrict__ vals) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sv[8]; __shared__ int si[8];
    const int r = blockIdx.x;
    float bv = -INFINITY; int bi = -1;
    for (int i = threadIdx.x; i < np; i += 256) am_better(bv, bi, pv[(size_t)r * np + i], pi[(size_t)r * np + i]);
    am_block_reduce(bv, bi, sv, si);
    if (threadIdx.x == 0) { ids[r] = bi; if (vals) vals[r] = bv; }
}
// ---- top-k per row (k <= TOPK_MAX), values descending, ties -> lower index (reference k_topk, ops.hip:702-716: k rounds
// of a masked arg-max). Stage 1: each block holds a chunk of the row in shared memory and extracts the chunk's own top k by
// k rounds of a block arg-max, masking each winner; stage 2 merges the np * k candidates of a row the same way. The k
// largest of the row are among the k largest of every chunk, so the result equals k rounds over the whole row.
constexpr int TOPK_MAX = 32;
__global__ void __launch_bounds__(256) k_topk_part(const float* __restrict__ x, int n, int ld, int k, float* __restrict__ pv, int* __restrict__ pi) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float buf[AM_CHUNK]; __shared__ float sv[8]; __shared__ int si[8]; __shared__ int s_win;
    const int r = blockIdx.y, c0 = blockIdx.x * AM_CHUNK, cn = min(n - c0, AM_CHUNK);
    const float* xr = x + (size_t)r * ld + c0;
    for (int i = threadIdx.x; i < cn; i += 256) buf[i] = xr[i];
    __syncthreads();
    for (int rd = 0; rd < k; ++rd) {
        float bv = -INFINITY; int bi = -1;
        for (int i = threadIdx.x; i < cn; i += 256) { const float v = buf[i]; if (v > bv) { bv = v; bi = c0 + i; } }
        am_block_reduce(bv, bi, sv, si);
        if (threadIdx.x == 0) { const size_t o = ((size_t)r * gridDim.x + blockIdx.x) * k + rd; pv[o] = bv; pi[o] = bi; s_win = bi; }
        __syncthreads();
        if (threadIdx.x == 0 && s_win >= 0) buf[s_win - c0] = -INFINITY;   // taken (an entry equal to -inf is never selected, as in the reference)
        __syncthreads();
    }
}
__global__ void __launch_bounds__(256) k_topk_final(const float* __restrict__ pv, const int* __restrict__ pi, int nc, int k, int* __restrict__ ids, float* __restrict__ vals) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float cv[64 * TOPK_MAX]; __shared__ int ci[64 * TOPK_MAX]; __shared__ float sv[8]; __shared__ int si[8]; __shared__ int s_win;
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < nc; i += 256) { cv[i] = pv[(size_t)r * nc + i]; ci[i] = pi[(size_t)r * nc + i]; }
    __syncthreads();
    for (int rd = 0; rd < k; ++rd) {
        float bv = -INFINITY; int bi = -1;
        for (int i = threadIdx.x; i < nc; i += 256) if (ci[i] >= 0) am_better(bv, bi, cv[i], ci[i]);
        am_block_reduce(bv, bi, sv, si);
        if (threadIdx.x == 0) { ids[(size_t)r * k + rd] = bi; if (vals) vals[(size_t)r * k + rd] = bv; s_win = bi; }
        __syncthreads();
        for (int i = threadIdx.x; i < nc; i += 256) if (ci[i] == s_win) ci[i] = -1;   // taken
        __syncthreads();
    }
}
// out[0] = mm (accepted drafts), out[1] = bonus token ids[mm]
__global__ void k_accept(const int* __restrict__ ids, const int* __restrict__ drafts, int n_draft, int* __restrict__ out) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int mm = 0; while (mm < n_draft && ids[mm] == drafts[mm]) ++mm;
        out[0] = mm; out[1] = ids[mm];
    }
}

// Scratch of the allocation-free entry point: partial (value, index) pairs for at most AM_STATIC_ROWS rows of at most
// AM_STATIC_PARTS * AM_CHUNK logits. It lives in the library image, so every GPU that loads the library holds these
// 16 KiB until the process exits. In host code the name below is only a handle for cudaGetSymbolAddress.
constexpr int AM_STATIC_ROWS = 32, AM_STATIC_PARTS = 64;
static __device__ __align__(256) unsigned char g_argmax_scratch[AM_STATIC_ROWS * AM_STATIC_PARTS * 8];
static void* g_argmax_scratch_addr[MAX_DEVICES] = {};   // per device ordinal; written without a lock (see the header: first call per device from one thread)

}  // namespace

size_t argmax_scratch_bytes(int R, int n) { return (size_t)R * ((n + AM_CHUNK - 1) / AM_CHUNK) * 8; }

int argmax_rows(const float* logits, int R, int n, int ld, int* ids, float* vals, void* scratch, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && n >= 1 && ld >= n && scratch, "argmax_rows: bad arguments R=%d n=%d ld=%d", R, n, ld);
    const int np = (n + AM_CHUNK - 1) / AM_CHUNK;
    float* pv = (float*)scratch; int* pi = (int*)(pv + (size_t)R * np);
    HP_CUDA(launch_pdl<1>(k_argmax_part, dim3(np, R), dim3(256), 0, s, logits, n, ld, pv, pi));
    HP_CUDA(launch_pdl<1>(k_argmax_final, dim3(R), dim3(256), 0, s, pv, pi, np, ids, vals));
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}
size_t topk_scratch_bytes(int R, int n, int k) { return (size_t)R * ((n + AM_CHUNK - 1) / AM_CHUNK) * k * 8; }
int topk_max_k() { return TOPK_MAX; }
int topk_rows(const float* logits, int R, int n, int ld, int k, int* ids, float* vals, void* scratch, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && n >= 1 && ld >= n && scratch && ids, "topk_rows: bad arguments R=%d n=%d ld=%d", R, n, ld);
    const int np = (n + AM_CHUNK - 1) / AM_CHUNK;
    HP_REQUIRE(k >= 1 && k <= TOPK_MAX && k <= n && np <= 64, "topk_rows: k=%d must be in 1..%d (and the row at most %d entries)", k, TOPK_MAX, 64 * AM_CHUNK);
    float* pv = (float*)scratch; int* pi = (int*)(pv + (size_t)R * np * k);
    HP_CUDA(launch_pdl<1>(k_topk_part, dim3(np, R), dim3(256), 0, s, logits, n, ld, k, pv, pi));
    HP_CUDA(launch_pdl<1>(k_topk_final, dim3(R), dim3(256), 0, s, (const float*)pv, (const int*)pi, np * k, k, ids, vals));
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}
int argmax_static_max_rows() { return AM_STATIC_ROWS; }
int argmax_static_max_n() { return AM_STATIC_PARTS * AM_CHUNK; }

// Same two kernels as argmax_rows, with the partials in the file-scope device array above instead of caller memory.
// The first call on a device looks the array's device address up (once per device, with that device current).
int argmax_rows_static(const float* logits, int R, int n, int ld, int* ids, float* vals, cudaStream_t s) {
    HP_REQUIRE(R >= 1 && n >= 1 && ld >= n, "argmax_rows_static: bad arguments R=%d n=%d ld=%d", R, n, ld);
    HP_REQUIRE(R <= AM_STATIC_ROWS && n <= AM_STATIC_PARTS * AM_CHUNK,
               "argmax_rows_static: R=%d n=%d exceed the built-in scratch (at most %d rows of %d entries)", R, n, AM_STATIC_ROWS, AM_STATIC_PARTS * AM_CHUNK);
    // The array whose address is needed is the copy on the device that owns the stream. A kernel can only be launched
    // into a stream of the current device, so a stream that belongs to another device is refused here rather than
    // handed the wrong device's address.
    const int cur = current_device();
    int dev = cur;
    if (s != nullptr && s != cudaStreamLegacy && s != cudaStreamPerThread) HP_CUDA(cudaStreamGetDevice(s, &dev));
    HP_REQUIRE(cur >= 0 && dev == cur, "argmax_rows_static: the stream belongs to device %d but device %d is current", dev, cur);
    if (!g_argmax_scratch_addr[dev]) {
        void* p = nullptr;
        HP_CUDA(cudaGetSymbolAddress(&p, g_argmax_scratch));
        g_argmax_scratch_addr[dev] = p;
    }
    const int np = (n + AM_CHUNK - 1) / AM_CHUNK;
    float* pv = (float*)g_argmax_scratch_addr[dev]; int* pi = (int*)(pv + (size_t)R * np);
    HP_CUDA(launch_pdl<1>(k_argmax_part, dim3(np, R), dim3(256), 0, s, logits, n, ld, pv, pi));
    HP_CUDA(launch_pdl<1>(k_argmax_final, dim3(R), dim3(256), 0, s, pv, pi, np, ids, vals));
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}

int accept_greedy(const int* ids, const int* drafts, int n_draft, int* out, cudaStream_t s) {
    HP_REQUIRE(n_draft >= 0 && n_draft <= 31, "accept_greedy: n_draft=%d out of range", n_draft);
    k_accept<<<1, 32, 0, s>>>(ids, drafts, n_draft, out);
    HP_CUDA(cudaGetLastError());
    return HP_OK;
}

}  // namespace hp
