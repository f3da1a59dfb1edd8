// Shared device helpers: status handling, deterministic fp32 math, Q4_K scale decode, mbarrier / bulk-copy PTX.
// Compiled with --fmad=false: every fused multiply-add in this code base is an explicit fmaf, so the rounding
// sequence of each kernel is fixed by its source and can be restated operation by operation on a CPU.
#pragma once
#include <cstdlib>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <string.h>

namespace hp {

// ---- status (never throw across the C boundary; reference: CK macro + std::runtime_error, engine/src/qwen35.cpp:10) ----
enum : int { HP_OK = 0, HP_EINVAL = 1, HP_ECUDA = 2, HP_ENOMEM = 3, HP_ETIMEOUT = 4, HP_ESTATE = 5, HP_ECOMM = 6 };
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);
#define HP_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) return hp::cuda_fail(e_, #x, __FILE__, __LINE__); } while (0)
#define HP_REQUIRE(cond, ...) do { if (!(cond)) { hp::set_error(__VA_ARGS__); return hp::HP_EINVAL; } } while (0)

// ---- deterministic exp / log: fixed sequences of IEEE fp32 operations (no fast intrinsics) ----
// The reference device code uses __expf / log1pf (engine/kernels/ops.hip:11-13); here they are defined so that
// a CPU can reproduce them bit for bit.
__host__ __device__ __forceinline__ float bits_f(uint32_t u) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}
__host__ __device__ __forceinline__ uint32_t f_bits(float f) {
#ifdef __CUDA_ARCH__
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
__host__ __device__ __forceinline__ float expf_det(float x) {
    float xc = x; if (xc > 90.f) xc = 90.f; if (xc < -110.f) xc = -110.f;
    const float fn = rintf(xc * 1.44269504088896341f);
    float r = fmaf(fn, -0.693359375f, xc);
    r = fmaf(fn, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    const float z = r * r;
    float y = fmaf(p, z, r) + 1.0f;
    const int n = (int)fn, n1 = n >> 1, n2 = n - n1;
    y = y * bits_f((uint32_t)(n1 + 127) << 23);
    return y * bits_f((uint32_t)(n2 + 127) << 23);
}
__host__ __device__ __forceinline__ float logf_ge1_det(float x) {
    const uint32_t ix = f_bits(x);
    int e = (int)(ix >> 23) - 127;
    float m = bits_f((ix & 0x007fffffu) | 0x3f800000u);
    if (m > 1.41421356237f) { m = m * 0.5f; e += 1; }
    const float f = m - 1.0f, z = f * f, fe = (float)e;
    float p = 7.0376836292e-2f;
    p = fmaf(p, f, -1.1514610310e-1f);
    p = fmaf(p, f, 1.1676998740e-1f);
    p = fmaf(p, f, -1.2420140846e-1f);
    p = fmaf(p, f, 1.4249322787e-1f);
    p = fmaf(p, f, -1.6668057665e-1f);
    p = fmaf(p, f, 2.0000714765e-1f);
    p = fmaf(p, f, -2.4999993993e-1f);
    p = fmaf(p, f, 3.3333331174e-1f);
    float y = (p * f) * z;
    y = fmaf(fe, -2.12194440e-4f, y);
    y = fmaf(z, -0.5f, y);
    const float r = f + y;
    return fmaf(fe, 0.693359375f, r);
}
__host__ __device__ __forceinline__ float log1pf_pos_det(float e) {
    const float u = 1.0f + e;
    if (u == 1.0f) return e;
    if (!(u < 3.0e38f)) return logf_ge1_det(3.0e38f);
    const float c = (e - (u - 1.0f)) / u;
    return logf_ge1_det(u) + c;
}
// ---- counter-based seeded generation: value = f(seed, stream id, index); integer arithmetic plus exactly rounded float
// operations only, so a CPU regenerates identical values ----
__host__ __device__ inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull; x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull; x = (x ^ (x >> 27)) * 0x94D049BB133111EBull; return x ^ (x >> 31);
}
__host__ __device__ inline uint64_t rnd64(uint64_t seed, uint64_t tid, uint64_t idx) { return splitmix64(splitmix64(seed ^ (tid * 0x9E3779B97F4A7C15ull)) + idx); }
__host__ __device__ inline float irwin(uint64_t u) {
    const int sum = (int)(u & 0xFFFF) + (int)((u >> 16) & 0xFFFF) + (int)((u >> 32) & 0xFFFF) + (int)(u >> 48) - 131070;
    return (float)sum * 2.6429e-5f;
}
__host__ __device__ __forceinline__ float sigmoid_det(float x) { return 1.0f / (1.0f + expf_det(-x)); }
__host__ __device__ __forceinline__ float silu_det(float x) { return x / (1.0f + expf_det(-x)); }
__host__ __device__ __forceinline__ float softplus_det(float x) { return x > 20.f ? x : log1pf_pos_det(expf_det(x)); }

#ifdef __CUDACC__
__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t f2h(float f) { return __half_as_ushort(__float2half_rn(f)); }
__device__ __forceinline__ float bf2f(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

// ---- Q4_K (144 B: f16 d, f16 dmin, 12 B of 6-bit scales/mins, 128 B of nibbles; engine/src/quant.h:22,37-40) ----
// hdr = the first 16 bytes of a block as a uint4. Returns the (scale, min) pair of sub-block sb (0..7).
__device__ __forceinline__ void q4k_scale_min(const uint4& hdr, int sb, uint32_t& sc, uint32_t& mn) {
    if (sb < 4) { sc = (hdr.y >> (8 * sb)) & 63u; mn = (hdr.z >> (8 * sb)) & 63u; }
    else {
        const int k = sb - 4;
        sc = ((hdr.w >> (8 * k)) & 0xFu) | (((hdr.y >> (8 * k + 6)) & 3u) << 4);
        mn = ((hdr.w >> (8 * k + 4)) & 0xFu) | (((hdr.z >> (8 * k + 6)) & 3u) << 4);
    }
}

// ---- mbarrier + bulk async copy (sm_90+/sm_100a) ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (hundreds of milliseconds), records the failure in *err and
// returns false; the caller stops issuing work and leaves the kernel.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err) {
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        if (mbar_test(bar, parity)) return true;
        if (it > 64) __nanosleep(it > 4096 ? 256 : 32);
    }
    if (err) atomicExch(err, hp::HP_ETIMEOUT);
    return false;
}
// 1-D bulk copy global -> shared of `bytes` (multiple of 16; both addresses 16-byte aligned), completion on mbarrier.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// 4-byte asynchronous copy global -> shared (Ampere-style cp.async); completion with cp_async_wait_all()
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// thread-block cluster: barrier over all threads of all CTAs (release / acquire), split arrive / wait, and a 32-bit
// store into the same shared-memory variable of CTA `rank` of the cluster
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_cluster_f32(float* local_smem, uint32_t rank, float v) {   // store into the same variable of CTA `rank`
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_smem)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
// programmatic dependent launch (no-ops when the kernel was not launched with the attribute)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch with the programmatic-dependent-launch attribute: the kernel may start while its predecessor in the stream is
// still running; it must execute pdl_wait() before touching anything the predecessor writes.
// Which kernel classes are launched WITHOUT the attribute (bit mask; class 0 counts as 32; the GEMV is 64). Measured on
// B200, class by class: in plain stream launches every class gains from the early launch; inside a captured CUDA graph the
// GEMV, the MoE kernels (work before the dependency wait: ring set-up, router rows), the SiLU kernel (-0.13 ms per dense
// round: its CTAs sit beside the gate|up GEMV's and start the moment it ends) and attention gain, while programmatic
// edges on the row norms and the GDN kernel cost ~0.1 ms per round each, so while a stream is being captured the default
// mask switches those and the bookkeeping classes off. HIPSTER_B200_PDL_OFF=<mask> overrides both.
inline int pdl_off_mask(cudaStream_t s) {
    static const int env = [] { const char* e = getenv("HIPSTER_B200_PDL_OFF"); return e ? atoi(e) : -1; }();
    if (env >= 0) return env;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &st) != cudaSuccess) return 0;
    return st == cudaStreamCaptureStatusActive ? 0x0B3 : 0;
}
template <int CLS = 0, typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = (pdl_off_mask(s) & (CLS ? CLS : 32)) ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- shared pieces of the Q4_K tensor-core GEMV inner loop (dense GEMV and routed-expert GEMV) ----
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(reinterpret_cast<unsigned long long&>(r))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return r;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(reinterpret_cast<unsigned long long&>(r))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return r;
}
// D = A * B + 0x4B400000 per element
__device__ __forceinline__ void mma_u8s8_magic(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0x4B400000));
}
__device__ __forceinline__ void fma2(float2& acc, float2 a, float2 b) {   // acc = a * b + acc, per lane, one rounding each
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(reinterpret_cast<unsigned long long&>(acc))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
}

// Scales of one row of one block: {d*sc, d*sc, -(dmin*mn), -(dmin*mn)} per sub-block, computed on demand.
struct RowScales {
    float d, cd, dq, cdq, nd, cnd;          // d, -(d*2^23), d/16, -(d/16*2^23), -dmin, dmin*2^23
    uint32_t sc[2], mn[2];                  // 6-bit scales / mins of sub-blocks 0-3 and 4-7, one per byte
    __device__ __forceinline__ float4 get(int k) const {
        const float fs = __uint_as_float(__byte_perm(sc[k >> 2], 0x4B000000u, 0x7540u | (k & 3)));
        const float fm = __uint_as_float(__byte_perm(mn[k >> 2], 0x4B000000u, 0x7540u | (k & 3)));
        const float s0 = (k & 1) ? fmaf(dq, fs, cdq) : fmaf(d, fs, cd);
        const float nm = fmaf(nd, fm, cnd);
        return make_float4(s0, s0, nm, nm);
    }
};
__device__ __forceinline__ RowScales decode_scales(const uint4 hdr) {
    RowScales r;
    r.d = h2f((uint16_t)(hdr.x & 0xFFFF)); r.nd = -h2f((uint16_t)(hdr.x >> 16));
    r.dq = r.d * 0.0625f;
    r.cd = -(r.d * 8388608.f); r.cdq = -(r.dq * 8388608.f); r.cnd = -(r.nd * 8388608.f);
    r.sc[0] = hdr.y & 0x3F3F3F3Fu; r.mn[0] = hdr.z & 0x3F3F3F3Fu;
    r.sc[1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
    r.mn[1] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
    return r;
}

// int8 tensor-core tile: D(16x8,s32) = A(16x32,u8 row) * B(32x8,s8 col) + 0
__device__ __forceinline__ void mma_u8s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}
#endif

// ---- activation layout consumed by the tensor-core GEMV ("fragment-major XQ8") ----
// Columns (= verify rows) are grouped in tiles of 8. For tile nt and 64-element group jj of K, lane (g = column in
// tile, t) owns 16 bytes: the 8 int8 of elements 64jj + 8t..8t+7 followed by the 8 int8 of elements 64jj+32+8t..+7,
// i.e. exactly its B fragments for the low-nibble and high-nibble sub-blocks of that group.
// Scales: per (tile, 32-element sub-block sb, column pair p) one float4 {d[2p], d[2p+1], s[2p], s[2p+1]}.
__host__ __device__ __forceinline__ size_t xq_tiles(int R) { return (size_t)(R + 7) / 8; }
__host__ __device__ __forceinline__ size_t xq_q_bytes(int R, int K) { return xq_tiles(R) * (size_t)K * 8; }
__host__ __device__ __forceinline__ size_t xq_sc_floats(int R, int K) { return xq_tiles(R) * (size_t)(K / 32) * 16; }
__host__ __device__ __forceinline__ size_t xq_q_index(int r, int k, int K) {
    const int nt = r >> 3, g = r & 7, jj = k >> 6, e = k & 63, sub = e >> 5, e32 = e & 31, t = e32 >> 3, byte = e32 & 7;
    return ((((size_t)nt * (K >> 6) + jj) * 32 + (g * 4 + t)) << 4) + sub * 8 + byte;
}
__host__ __device__ __forceinline__ size_t xq_d_index(int r, int sb, int K) {
    const int nt = r >> 3, g = r & 7;
    return ((((size_t)nt * (K >> 5) + sb) * 4 + (g >> 1)) << 2) + (g & 1);
}   // the matching s is at +2

#ifdef __CUDACC__
// One warp quantises 32 consecutive activations (lane-owned value v) of verify row r, sub-block sb, into the
// fragment-major layout: amax over 32; d = amax/127; id = 127/amax (two separate divisions); q = rint(v*id)
// (round-half-even); s = d * sum(q). Reference: k_quantize_x_q8 / wave_quant32 (gemv.hip:36-51, ops.hip:49-60).
__device__ __forceinline__ void warp_quant32_store(float v, int r, int sb, int K, int8_t* __restrict__ q, float* __restrict__ sc, int lane) {
    float amax = fabsf(v);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float dd = amax / 127.f, id = amax > 0.f ? 127.f / amax : 0.f;
    const int qi = __float2int_rn(v * id);
    int sum = qi;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    q[xq_q_index(r, sb * 32 + lane, K)] = (int8_t)qi;
    if (lane == 0) { const size_t di = xq_d_index(r, sb, K); sc[di] = dd; sc[di + 2] = dd * (float)sum; }
}
#endif

}  // namespace hp
