// Lightning-indexer scores on tcgen05: score[key] = sum over index heads of relu(q_h . k) * w_h.
//
// Reference counterparts: glm53/gfx950/kernel.py:2739-2997 (index score in f32 over bf16 operands);
// FP4 index keys with one E8M0 code per 32 dims as deepseek_v4/gfx950/kernels/stages/indexer.py:143-151.
//
// One CTA of 128 threads takes a run of 128-key tiles of one row.  The keys are the M side of the MMA
// (key i of a tile = TMEM lane i = thread i of the CTA), the index heads the N side (64 columns), the
// 128 dims the K side: after one tcgen05.ld a thread holds the 64 head dots of ITS key, so the
// relu-weighted sum over heads is 64 FMAs inside the thread with no shuffles, and the operands are
// read from shared memory once by the tensor core instead of once per warp.
//   thread i: FP4 key -> bf16 (exact: E2M1 x 2^(code-127)) -> row i of the A tile (128-byte swizzle)
//   thread 0: 8 x tcgen05.mma kind::f16 (M 128, N 64, K 16) -> 64 TMEM columns, commit -> mbarrier
//   thread i: tcgen05.ld of lane i, sum, store.  Two A buffers and two accumulators alternate, so the
//   conversion of tile t+1 and the sum of tile t-1 run while the MMAs of tile t are in flight.
#include <cstdlib>
#include "mono_common.cuh"

extern void mono_set_error(const char* fmt, ...);

namespace mono {
namespace isc {

constexpr int kThreads = 128;
constexpr int kTile = 128;                 // keys per tile
constexpr int kABytes = kTile * 256;       // one A buffer: 128 keys x 128 bf16, as two 64-dim halves of 16 KB
constexpr int kBBytes = 64 * 256;          // q: 64 heads x 128 bf16, as two 64-dim halves of 8 KB
constexpr int kSmemBytes = 1024 + 2 * kABytes + kBBytes;
constexpr uint32_t kTmemCols = 128;        // two accumulators of 64 columns
constexpr int kMaxTilesPerTask = 32;
// instruction descriptor: D f32, A and B bf16, both K-major, N = 64, M = 128
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    // K-major rows of 128 bytes, 128-byte swizzle, groups of 8 rows 1024 bytes apart
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate)
        : "memory");
}
// byte offset of 16-byte chunk `ch` (0..15 over the 128 dims) of row r inside an operand whose two
// 64-dim halves are `half_bytes` apart
__device__ __forceinline__ uint32_t swz(int r, int ch, uint32_t half_bytes) {
    return (uint32_t)(ch >> 3) * half_bytes + (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u +
           (uint32_t)(((ch & 7) ^ (r & 7)) << 4);
}

struct RawKey {
    uint4 v[4];
    uint32_t codes;
};

// `pages`: the page table entries of the task's keys (shared memory), entry 0 = the page of key p0
__device__ __forceinline__ RawKey request_key(const mono_index_args& a, const int* pages, int p0, int p, int n) {
    RawKey k;
    k.v[0] = k.v[1] = k.v[2] = k.v[3] = make_uint4(0, 0, 0, 0);
    k.codes = 0x7f7f7f7fu;
    if (p < n) {
        const int64_t pg = pages[(p - p0) / kPage];
        if (pg >= 0 && pg < a.n_pages) {
            const uint8_t* page = a.idx_pages + (size_t)pg * kIdxPageBytes;
            const int off = p % kPage;
            const uint4* src = reinterpret_cast<const uint4*>(page + (size_t)off * 64);
#pragma unroll
            for (int i = 0; i < 4; ++i) k.v[i] = __ldg(src + i);
            k.codes = __ldg(reinterpret_cast<const uint32_t*>(page + kPage * 64 + off * 4));
        }
    }
    return k;
}

// One row of the A tile: 128 E2M1 codes (16 words) and 4 scale codes -> 16 chunks of 8 bf16.
__device__ __forceinline__ void store_key(uint8_t* abuf, int r, const RawKey& k) {
    const uint32_t w[16] = {k.v[0].x, k.v[0].y, k.v[0].z, k.v[0].w, k.v[1].x, k.v[1].y, k.v[1].z, k.v[1].w,
                            k.v[2].x, k.v[2].y, k.v[2].z, k.v[2].w, k.v[3].x, k.v[3].y, k.v[3].z, k.v[3].w};
#pragma unroll
    for (int wi = 0; wi < 16; ++wi) {
        // the block scale 2^(code - 127) as two bf16 (code 0 reads as 1, like the oracle): its product
        // with an E2M1 value is exact in bf16
        const uint32_t code = max((k.codes >> ((wi >> 2) * 8)) & 0xFFu, 1u);
        const uint32_t sc2 = (code << 7) | (code << 23);
        // E2M1 magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6 as bf16: a byte permute looks up the high and the low
        // bytes of four codes at once (the 3 magnitude bits of a nibble are its selector), two more
        // interleave them into bf16 pairs, and the sign bit of each nibble moves to bit 15 of its half
        uint32_t o[4];
#pragma unroll
        for (int hw = 0; hw < 2; ++hw) {
            const uint32_t w16 = hw ? w[wi] >> 16 : w[wi];
            const uint32_t sel = w16 & 0x7777u;
            const uint32_t hb = __byte_perm(0x3F3F3F00u, 0x40404040u, sel);
            const uint32_t lb = __byte_perm(0xC0800000u, 0xC0804000u, sel);
            const uint32_t p01 = __byte_perm(lb, hb, 0x5140) | ((w16 << 12) & 0x8000u) | ((w16 << 24) & 0x80000000u);
            const uint32_t p23 = __byte_perm(lb, hb, 0x7362) | ((w16 << 4) & 0x8000u) | ((w16 << 16) & 0x80000000u);
            const __nv_bfloat162 r01 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&p01), *reinterpret_cast<const __nv_bfloat162*>(&sc2));
            const __nv_bfloat162 r23 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&p23), *reinterpret_cast<const __nv_bfloat162*>(&sc2));
            o[2 * hw] = *reinterpret_cast<const uint32_t*>(&r01);
            o[2 * hw + 1] = *reinterpret_cast<const uint32_t*>(&r23);
        }
        *reinterpret_cast<uint4*>(abuf + swz(r, wi, kABytes / 2)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

__device__ __forceinline__ void ld64(uint32_t taddr, uint32_t r[64]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]), "+r"(r[32]), "+r"(r[33]), "+r"(r[34]), "+r"(r[35]), "+r"(r[36]), "+r"(r[37]), "+r"(r[38]), "+r"(r[39]), "+r"(r[40]), "+r"(r[41]), "+r"(r[42]), "+r"(r[43]), "+r"(r[44]), "+r"(r[45]), "+r"(r[46]), "+r"(r[47]), "+r"(r[48]), "+r"(r[49]), "+r"(r[50]), "+r"(r[51]), "+r"(r[52]), "+r"(r[53]), "+r"(r[54]), "+r"(r[55]), "+r"(r[56]), "+r"(r[57]), "+r"(r[58]), "+r"(r[59]), "+r"(r[60]), "+r"(r[61]), "+r"(r[62]), "+r"(r[63])
                 :
                 : "memory");
}

// NB = 2: two A buffers and accumulators per CTA (two CTAs per SM); NB = 1: one of each (four CTAs per SM,
// the overlap comes from the other CTAs of the SM).
template <int NB>
__global__ void __launch_bounds__(kThreads) index_score_tc_kernel(const mono_index_args a, int max_tiles, int tiles_per_task) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* abuf = smem;                // two A buffers
    uint8_t* bbuf = smem + NB * kABytes;  // q
    __shared__ float w[64];
    __shared__ __align__(8) uint64_t mma_done[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_flag;
    __shared__ int pages[kMaxTilesPerTask * (kTile / kPage)];
    const int tid = threadIdx.x, warp = tid >> 5;
    const int groups = (max_tiles + tiles_per_task - 1) / tiles_per_task;
    const int row = blockIdx.x / groups, tile0 = (blockIdx.x - row * groups) * tiles_per_task;
    pdl_launch_dependents();
    // ---- set-up that does not read what the launch before this one wrote
    if (tid == 0) {
        abort_flag = 0;
        mbar_init(&mma_done[0], 1);
        mbar_init(&mma_done[1], 1);
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(64u * NB) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = tmem_base_s;
    {
        // during the wait for the launch that writes the index queries: the row's head weights (written
        // by an earlier launch; an L2 prefetch is safe in any case) and the bytes of this thread's first key
        // (the step's positions, slots and page table are inputs of the step; the index key of the new
        // token was written launches ago)
        if (tid == 0) prefetch_l2(a.idx_w + (size_t)row * a.w_ld);
        const int p = tile0 * kTile + tid;
        const int pi = p / kPage;
        if (pi < a.pt_ld && (!a.slots || a.slots[row] >= 0) && p <= (int)a.positions[row]) {
            const int64_t pg = a.page_table[(size_t)row * a.pt_ld + pi];
            if (pg >= 0 && pg < a.n_pages) {
                const uint8_t* page = a.idx_pages + (size_t)pg * kIdxPageBytes;
                prefetch_l2(page + (size_t)(p % kPage) * 64);
                if ((tid & 31) == 0) prefetch_l2(page + kPage * 64 + (p % kPage) * 4);
            }
        }
    }
    pdl_wait();
    // the row's position, its slot and the task's page table entries are requested together (one memory
    // latency); a key request is then one more, not two
    const int p0 = tile0 * kTile;
    int my_page = -1;
    if (tid < tiles_per_task * (kTile / kPage)) {
        const int pi = p0 / kPage + tid;
        if (pi < a.pt_ld) my_page = a.page_table[(size_t)row * a.pt_ld + pi];
    }
    const int64_t slot = a.slots ? a.slots[row] : 0;
    const int64_t pos = a.positions[row];
    if (tid < tiles_per_task * (kTile / kPage)) pages[tid] = my_page;
    const int n = slot >= 0 ? (int)pos + 1 : 0;
    const int ntile = min(tiles_per_task, (n + kTile - 1) / kTile - tile0);  // <= 0: nothing to do
    if (ntile > 0) {
        __syncthreads();
        RawKey nk = request_key(a, pages, p0, p0 + tid, n);
        // ---- q (zero rows past index_heads) as the B operand, and the head weights
        if (a.iq) {
            // the queries are made here from the q_b GEMV's partial sums: a warp takes a head at a time, a lane
            // dims 4 lane .. 4 lane + 3.  Sum of the slices, interleaved RoPE on dims 0..63, Hadamard
            // butterflies of span 1, 2, 4 ... 64 (spans 1 and 2 inside the lane, the others by shuffles),
            // x 128^-1/2: the arithmetic and its order are those of the stand-alone query stage.
            const int lane = tid & 31;
            const __nv_bfloat16* cosb = reinterpret_cast<const __nv_bfloat16*>(a.cos);
            const __nv_bfloat16* sinb = reinterpret_cast<const __nv_bfloat16*>(a.sin);
            float c0 = 0.f, s0 = 0.f, c1 = 0.f, s1 = 0.f;
            if (lane < 16) {
                c0 = __bfloat162float(cosb[pos * 32 + 2 * lane]);
                s0 = __bfloat162float(sinb[pos * 32 + 2 * lane]);
                c1 = __bfloat162float(cosb[pos * 32 + 2 * lane + 1]);
                s1 = __bfloat162float(sinb[pos * 32 + 2 * lane + 1]);
            }
            __nv_bfloat16* qout = (a.idx_q && tile0 == 0) ? reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(a.idx_q)) : nullptr;
#pragma unroll 2
            for (int h = warp; h < 64; h += kThreads / 32) {
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (h < a.index_heads) {
                    const float* src = a.iq + (size_t)row * a.iq_ld + h * 128 + 4 * lane;
                    for (int sl = 0; sl < a.iq_nsum; ++sl) {
                        const float4 p = *reinterpret_cast<const float4*>(src + (size_t)sl * a.iq_sum_stride);
                        v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
                    }
                    if (lane < 16) {
                        const float x0 = v[0], x1 = v[1], x2 = v[2], x3 = v[3];
                        v[0] = x0 * c0 - x1 * s0;
                        v[1] = x0 * s0 + x1 * c0;
                        v[2] = x2 * c1 - x3 * s1;
                        v[3] = x2 * s1 + x3 * c1;
                    }
                    {   // span 1, then span 2
                        const float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
                        v[0] = a0 + a2; v[2] = a0 - a2; v[1] = a1 + a3; v[3] = a1 - a3;
                    }
#pragma unroll
                    for (int m = 1; m < 32; m <<= 1) {  // span 4 m: the partner is lane ^ m
                        const bool upper = (lane & m) != 0;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
                            v[j] = upper ? o - v[j] : v[j] + o;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] *= 0.08838834764831845f;
                }
                const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
                const uint2 pk = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
                *reinterpret_cast<uint2*>(bbuf + swz(h, lane >> 1, kBBytes / 2) + (lane & 1) * 8) = pk;
                if (qout && h < a.index_heads) *reinterpret_cast<uint2*>(qout + ((size_t)row * a.index_heads + h) * 128 + 4 * lane) = pk;
            }
        } else {
            const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(a.idx_q);
            uint4 qv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = tid + i * kThreads, h = c >> 4, ch = c & 15;
                qv[i] = make_uint4(0, 0, 0, 0);
                if (h < a.index_heads) qv[i] = *reinterpret_cast<const uint4*>(qg + ((size_t)row * a.index_heads + h) * 128 + ch * 8);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = tid + i * kThreads;
                *reinterpret_cast<uint4*>(bbuf + swz(c >> 4, c & 15, kBBytes / 2)) = qv[i];
            }
        }
        if (tid < 64) w[tid] = tid < a.index_heads ? a.idx_w[(size_t)row * a.w_ld + tid] : 0.f;
        const uint32_t a_addr = smem_u32(abuf), b_addr = smem_u32(bbuf);
        const uint32_t tmem_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
        // sum over heads of relu(dot) * w for tile t, whose MMAs were committed to mma_done[t & 1]
        auto finish = [&](int t) {
            const int buf = NB == 2 ? t & 1 : 0;
            const bool ok = mbar_wait(&mma_done[buf], (uint32_t)(NB == 2 ? t >> 1 : t) & 1u, &abort_flag);
            fence_after();
            float s = __int_as_float(0x7fc00000);  // a wait that ran out leaves a NaN, never a plausible score
            if (ok) {
                uint32_t d[64];
                ld64(tmem_lane + buf * 64, d);
                s = 0.f;
#pragma unroll
                for (int h = 0; h < 64; ++h) s += fmaxf(__uint_as_float(d[h]), 0.f) * w[h];
            }
            const int p = (tile0 + t) * kTile + tid;
            if (p < n) a.scores[(size_t)row * a.score_ld + p] = s;
            fence_before();
        };
#pragma unroll 1
        for (int t = 0; t < ntile; ++t) {
            const int buf = NB == 2 ? t & 1 : 0;
            store_key(abuf + buf * kABytes, tid, nk);
            if (t + 1 < ntile) nk = request_key(a, pages, p0, (tile0 + t + 1) * kTile + tid, n);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these stores before the tensor core's reads
            __syncthreads();
            if (tid == 0) {
                fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    // 16 dims = 32 bytes per MMA: four steps inside a 64-dim half, then the other half
                    const uint64_t ad = desc_sw128(a_addr + buf * kABytes + (ks >> 2) * (kABytes / 2)) + 2 * (ks & 3);
                    const uint64_t bd = desc_sw128(b_addr + (ks >> 2) * (kBBytes / 2)) + 2 * (ks & 3);
                    mma_bf16(tmem_base + buf * 64, ad, bd, ks ? 1u : 0u);
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&mma_done[buf])) : "memory");
            }
            if (NB == 1) {
                finish(t);
                __syncthreads();  // every thread has read the accumulator before the next tile's MMAs
            } else if (t > 0) {
                finish(t - 1);
            }
        }
        if (NB == 2) finish(ntile - 1);
    }
    fence_before();
    __syncthreads();
    if (warp == 0) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(64u * NB) : "memory");
    }
}

}  // namespace isc
}  // namespace mono

// Launches the tcgen05 score kernel for arguments mono_index_score_launch has validated.
int mono_index_score_tc_launch(const mono_index_args* a, void* stream) {
    using namespace mono;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        cudaError_t e = cudaFuncSetAttribute(isc::index_score_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, isc::kSmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(isc::index_score_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, isc::kSmemBytes - isc::kABytes);
        if (e != cudaSuccess) return (int)e;
        mono::attr_done(attr_once);
    }
    const char* nbs = getenv("MONO_ISC_BUFS");
    const int nb = nbs && nbs[0] == '1' ? 1 : 2;
    const int max_tiles = (a->score_ld + isc::kTile - 1) / isc::kTile;
    const int sms = mono_sm_count();
    // every CTA resident at once (two or four per SM): as many tiles per CTA as that takes
    const long resident = (nb == 2 ? 2L : 4L) * sms;
    int per = (int)(((long)a->rows * max_tiles + resident - 1) / resident);
    if (per < 1) per = 1;
    if (const char* f = getenv("MONO_ISC_TILES")) per = atoi(f) > 0 ? atoi(f) : per;
    if (per > isc::kMaxTilesPerTask) per = isc::kMaxTilesPerTask;  // more CTAs than are resident at once: they queue
    const int groups = (max_tiles + per - 1) / per;
    if (nb == 2)
        launch_k(isc::index_score_tc_kernel<2>, a->rows * groups, isc::kThreads, isc::kSmemBytes, (cudaStream_t)stream, *a, max_tiles, per);
    else
        launch_k(isc::index_score_tc_kernel<1>, a->rows * groups, isc::kThreads, isc::kSmemBytes - isc::kABytes, (cudaStream_t)stream, *a, max_tiles, per);
    return (int)cudaGetLastError();
}
