// Common device runtime of the sm_100a decoder-layer kernels: guard words and
// bounded waits, mbarrier / TMA / bulk-copy wrappers, MMA wrappers, number formats.
//
// Counterpart of the reference's common/ package (common/sync.py bounded spin,
// common/guard.py sticky error words, common/ops.py wave primitives, common/mx.py
// FP8 / MX helpers), rebuilt on mbarriers, TMA and warp-level MMA.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mono_b200.h"

namespace mono {

constexpr int kPage = MONO_PAGE_TOKENS;
constexpr int kKvDim = MONO_KV_DIM;
constexpr int kKvPageBytes = MONO_KV_PAGE_BYTES;
constexpr int kIdxPageBytes = MONO_IDX_PAGE_BYTES;
constexpr int kMaxRows = MONO_MAX_ROWS;

// ------------------------------------------------------------------ guard
// Guard words (int32[MONO_GUARD_WORDS]) follow common/guard.py:59-60,100-241: word 0
// is the epoch, words 3..5 are sticky error words, words 8.. are the flag words peers
// write.  A wait that runs out stores site + 1 into MONO_ERR_DEADLINE; every later
// wait sees a non-zero error word and returns at once, so the launch drains and the
// host reads the words.  Nothing traps.
__device__ __forceinline__ bool guard_failed(const int* g) {
    if (g == nullptr) return false;
    const volatile int* v = g;
    return (v[MONO_ERR_DEADLINE] | v[MONO_ERR_PEER] | v[MONO_ERR_ARG]) != 0;
}
__device__ __forceinline__ void guard_fail(int* g, int word, int site) {
    if (g != nullptr) atomicCAS(g + word, 0, site + 1);
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the time limit ran out or another thread aborted.  The
// default limit is generous (2 s): it exists so that no launch can hang a GPU.  Launches
// whose argument block carries a deadline (mono_gemv_args.wait_ns, set from the build
// context's deadline_s as the reference ties its deadline to the server's watchdog,
// common/guard.py:4-7,69) pass it as `limit_ns`.
constexpr uint64_t kWaitLimitNs = 2000000000ull;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t limit_ns = kWaitLimitNs) {
    // a try_wait suspends the thread for a hardware-defined interval: a few of them cover the usual wait,
    // and the (slow) global timer is only read once a wait is clearly long
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 15) == 15) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > limit_ns) break;
        }
    }
    *abort_flag = 1;
    return false;
}

// ------------------------------------------------------------------ TMA / bulk copies
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2),
        "r"(smem_u32(bar))
        : "memory");
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ------------------------------------------------------------------ shared loads
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// ------------------------------------------------------------------ MMA (warp level)
// D(16x8,f32) += A(16x32,e4m3,row) * B(32x8,e4m3,col)
__device__ __forceinline__ void mma_e4m3(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t r[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t r[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t r[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t r[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// ------------------------------------------------------------------ warp / block reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block sum in a fixed order (warp butterflies, then warp partials added in warp
// order by every thread), so that every block computes bit-identical results.
template <int WARPS>
__device__ __forceinline__ float block_sum(float v, float* red /* [WARPS] */) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < WARPS; ++i) s += red[i];
    return s;
}
template <int WARPS>
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = red[0];
#pragma unroll
    for (int i = 1; i < WARPS; ++i) s = fmaxf(s, red[i]);
    return s;
}

// ------------------------------------------------------------------ number formats
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint8_t f32_to_e4m3(float x) {
    return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}
// Biased exponent of the smallest power of two >= v (v > 0 finite): exponent +
// (mantissa != 0).  common/mx.py:27-39.
__device__ __forceinline__ int code_ceil(float v) {
    uint32_t b = __float_as_uint(v);
    return (int)((b >> 23) & 0xFF) + ((b & 0x7FFFFF) != 0 ? 1 : 0);
}
__device__ __forceinline__ float exp2_code(int code) {  // 2^(code-127), code in 1..254
    return __uint_as_float((uint32_t)code << 23);
}
// E2M1 code (0..15) of a float by saturating round-to-nearest-even.
__device__ __forceinline__ uint32_t f32_to_e2m1(float v) {
    float a = fabsf(v);
    uint32_t c = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
    return c | ((__float_as_uint(v) >> 28) & 8u);
}
__device__ __forceinline__ float e2m1_to_f32(uint32_t c) {
    const float lut[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    float m = lut[c & 7];
    return (c & 8) ? -m : m;
}

// ------------------------------------------------------------------ programmatic dependent launch
// Every kernel lets its successor start early (prologue, and for the GEMV kernel the
// first weight tiles, overlap this kernel's tail) and waits for its predecessors before
// it touches anything they wrote or still read.  Without the launch attribute both
// instructions do nothing.  This is how weight loads are issued ahead of upstream
// results across launch boundaries (the reference does it inside one kernel: each task
// issues its weight loads before it polls its inputs, glm53/gfx950/kernel.py:24-27,649-694).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Sum of `nsum` partial results `stride` floats apart, in the order s = 0, 1, ...  The loads of a batch of B are
// issued together, so a sum costs one memory round trip per batch rather than one per partial: every load of a
// batch is unconditional (entries past the last repeat the last partial's address and add +0, which changes no
// bit of a sum that starts at +0): a load whose only use sits under a condition is moved down into it, behind
// the additions before it.
// A 16-byte L2 load that keeps its place in program order among its kind (the compiler neither delays it to its
// first use nor drops it into a branch): what lets a batch of loads be in flight together.
__device__ __forceinline__ float4 ld_cg_f4_ordered(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
template <int B>
__device__ __forceinline__ float4 sum_partials4(const float* p, size_t stride, int nsum) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < nsum; s0 += B) {
        float4 t[B];
#pragma unroll
        for (int j = 0; j < B; ++j)
            t[j] = ld_cg_f4_ordered(p + (size_t)min(s0 + j, nsum - 1) * stride);
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const bool on = s0 + j < nsum;  // a select on the value: the load itself stays unconditional
            v.x += on ? t[j].x : 0.f; v.y += on ? t[j].y : 0.f; v.z += on ? t[j].z : 0.f; v.w += on ? t[j].w : 0.f;
        }
    }
    return v;
}
template <int B>
__device__ __forceinline__ float2 sum_partials2(const float* p, size_t stride, int nsum) {
    float2 v = make_float2(0.f, 0.f);
    for (int s0 = 0; s0 < nsum; s0 += B) {
        float2 t[B];
#pragma unroll
        for (int j = 0; j < B; ++j)
            t[j] = __ldcg(reinterpret_cast<const float2*>(p + (size_t)min(s0 + j, nsum - 1) * stride));
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const bool on = s0 + j < nsum;
            v.x += on ? t[j].x : 0.f; v.y += on ? t[j].y : 0.f;
        }
    }
    return v;
}

__device__ __forceinline__ void pdl_prologue() {
    pdl_launch_dependents();
    pdl_wait();
}
// What a kernel may do before pdl_wait(): under programmatic dependent launch its CTAs start while the
// launch before it still runs, so only data that launch does not write may be touched.  Between two
// layers' weight streams nothing of a small kernel's tables is left in L2: pulling them in during the
// wait takes their HBM latency off the dependent chain.  A prefetch into L2 is safe for any address
// (L2 is the device's point of coherence), which is why these helpers do nothing else.
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// the threads tid = 0 .. nthreads-1 pull `bytes` bytes at p into L2, one 128-byte line per thread and turn
__device__ __forceinline__ void prefetch_span(const void* p, size_t bytes, int tid, int nthreads) {
    if (!p) return;
    const char* c = reinterpret_cast<const char*>(p);
    for (size_t o = (size_t)tid * 128; o < bytes; o += (size_t)nthreads * 128) prefetch_l2(c + o);
}

// ld / st that bypass the non-coherent L1 (data produced by other SMs or other GPUs)
__device__ __forceinline__ float ld_cg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

}  // namespace mono

// ------------------------------------------------------------------ timeline stamps
// Built with -DMONO_TIMELINE (MONO_TIMELINE=1 in the environment of the build script), a kernel records the
// global timer at numbered points, per CTA, into a per-file device array that mono_timeline_read copies out
// (the reference's SGLANG_AMD_MONO_TIMELINE stamps: common/stamps.py:16-33, 48 points per CTA there).
// Without the flag the macros expand to nothing.
#ifdef MONO_TIMELINE
#define MONO_TL_POINTS 16
#define MONO_TL_CTAS 160
#define MONO_TL_DECLARE(name) static __device__ unsigned long long name[MONO_TL_CTAS][MONO_TL_POINTS];
#define MONO_TL(name, p)                                                                                         \
    do {                                                                                                         \
        if (threadIdx.x == 0 && blockIdx.x < MONO_TL_CTAS && (p) < MONO_TL_POINTS) name[blockIdx.x][p] = mono::globaltimer_ns(); \
    } while (0)
// the same from any one thread the caller has picked (e.g. lane 0 of a role's warp)
#define MONO_TL_AT(name, p)                                                                                      \
    do {                                                                                                         \
        if (blockIdx.x < MONO_TL_CTAS && (p) < MONO_TL_POINTS) name[blockIdx.x][p] = mono::globaltimer_ns();     \
    } while (0)
#else
#define MONO_TL_DECLARE(name)
#define MONO_TL(name, p) do { } while (0)
#define MONO_TL_AT(name, p) do { } while (0)
#endif

// Host side: one launch helper, with or without the programmatic-serialization attribute.
#include <atomic>
extern int g_mono_pdl;
extern std::atomic<unsigned long long> g_mono_launches;  // kernels launched through launch_k since the library was loaded
namespace mono {
// Function attributes (the > 48 KB dynamic shared memory opt-in) belong to a device's copy of a
// kernel, so they are set once per device, whichever thread first launches there.  Usage:
//   static std::atomic<uint64_t> once{0};
//   if (attr_needed(once)) { ... cudaFuncSetAttribute ...; if ok: attr_done(once); }
inline int current_device_bit(uint64_t* bit) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev > 63) return -1;
    *bit = 1ull << dev;
    return dev;
}
inline bool attr_needed(const std::atomic<uint64_t>& once) {
    uint64_t bit = 0;
    if (current_device_bit(&bit) < 0) return true;
    return (once.load(std::memory_order_acquire) & bit) == 0;
}
inline void attr_done(std::atomic<uint64_t>& once) {
    uint64_t bit = 0;
    if (current_device_bit(&bit) >= 0) once.fetch_or(bit, std::memory_order_release);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = g_mono_pdl ? 1 : 0;
    g_mono_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}
}  // namespace mono
