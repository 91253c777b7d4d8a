// Weight-streaming GEMV on 5th-generation tensor cores: tcgen05.mma (kind::f8f6f4) with the
// accumulators in tensor memory, both operands fed by TMA.
//
// Same contract, task list and arithmetic as gemv.cu (reference: the MFMA GEMV units of
// glm53/gfx950/kernel.py:1061-1172 and the block-scale rule of :35-42): the 128 weight rows of
// a task are the MMA's M dimension, the step's rows (padded to 16) its N dimension; every 128-k
// chunk is accumulated on its own in TMEM and multiplied by the 128x128 weight scale and the
// per-row activation scale when the epilogue folds it into the task's f32 sum.
//
// Warp roles (192 threads): warp 0 issues the TMA loads of a stage (one 128 x 128-byte weight box
// and one 16 x 128-byte box per activation plane, all with the 128-byte swizzle, which is exactly
// the K-major shared-memory layout tcgen05 reads); one thread of warp 1 issues the MMAs and commits
// them to the stage's "free" barrier and the accumulator's "full" barrier; warps 2..5 own the 128
// TMEM lanes (one weight row per thread), read a finished accumulator with tcgen05.ld, scale and add.
#include "mono_common.cuh"
#include <cstdlib>
#include <mutex>
#include <vector>

extern void mono_set_error(const char* fmt, ...);

namespace mono {
MONO_TL_DECLARE(tl_gemv)

constexpr int kTcThreads = 320;  // TMA, MMA, 4 epilogue warps, 4 finisher warps
// A pipeline unit is kTcUnit k tiles: one barrier round trip, one commit, one TMEM load for all of them.  A stage
// holds a unit's weight tiles and its tiles of each activation plane, and feeds its own accumulators.
constexpr int tc_stages(int unit) { return unit == 4 ? 3 : unit == 2 ? 5 : 8; }
constexpr int kTcBarStages = 8;  // barrier slots (the larger stage count)
constexpr int kTcABytes = 128 * 128;
constexpr int kTcBBytes = 16 * 128;
constexpr int tc_tmem_cols(int unit) { return unit >= 2 ? 256 : 128; }  // stages x unit x 16 columns, a power of two
constexpr int kTcMaxSegTiles = 32;
constexpr int kTcListCache = 128;  // expert-list entries per job kept in shared memory
constexpr int kTcScSlotsMax = 4;  // segments whose scales may be in flight
constexpr int tc_sc_slots(int unit) { return unit == 4 ? 2 : 4; }  // (the four-tile unit needs the room for its stages)
constexpr int kTcScRows = 18;  // 16 activation-scale rows, the weight scales, the row coefficients

struct TcParams {
    mono_gemv_args a;
    int stages, stage_bytes;
    int prefetch_tiles;  // weight tiles each CTA pulls towards L2 while the launch before it drains
};

struct TcSeg {
    int c2, row0, t0, nt, aset;  // aset: activation set (head / expert slot) of the segment
    const float* asc;
    const float* wsc;
    const float* coef;
};

__device__ __forceinline__ int tc_nrb(const mono_gemv_job& j) {
    return (j.mode == MONO_JOB_DENSE && j.rb_per_mat > 0) ? j.n_mats * j.rb_per_mat : (j.n_rows + 127) >> 7;
}

__device__ __forceinline__ TcSeg tc_make_seg(const mono_gemv_job& j, int rb, int ks, int u, const int* elist = nullptr) {
    TcSeg s;
    int mat = 0, rbm = rb;
    if (j.mode == MONO_JOB_DENSE) {
        if (j.rb_per_mat > 0) { mat = rb / j.rb_per_mat; rbm = rb - mat * j.rb_per_mat; }
        s.t0 = ks * j.split_tiles;
        s.nt = min(j.split_tiles, j.k_tiles - s.t0);
        s.aset = j.act_seg_stride ? mat : 0;
        s.coef = nullptr;
    } else if (j.mode == MONO_JOB_EXPERT_UP) {
        mat = (elist && u < kTcListCache) ? elist[u] : j.expert_list[u];
        s.t0 = ks * j.split_tiles;
        s.nt = min(j.split_tiles, j.k_tiles - s.t0);
        s.aset = 0;
        s.coef = nullptr;
    } else {
        mat = (elist && u < kTcListCache) ? elist[u] : j.expert_list[u];
        s.t0 = 0;
        s.nt = j.k_tiles;
        s.aset = u;
        s.coef = j.coef ? j.coef + (size_t)u * kMaxRows : nullptr;
    }
    s.c2 = mat;
    s.row0 = j.row_off + rbm * 128;
    s.asc = j.ascale_f32 + (size_t)s.aset * j.ascale_seg_stride + s.t0;
    s.wsc = j.wscale_f32 + (size_t)mat * j.wscale_mat_stride + (size_t)(s.row0 >> 7) * j.wscale_ld + s.t0;
    return s;
}

// ---- tcgen05 wrappers
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], kind::f8f6f4, one CTA
__device__ __forceinline__ void tc_mma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// TMEM -> registers in two steps, so that the load of the next accumulators can be in flight during the
// math on these.  The wait names the registers as in/out operands: no read of them may move above it.
// 32 columns (two accumulators) at once
__device__ __forceinline__ void tc_ld32_issue(uint32_t taddr, uint32_t r[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tc_ld32_wait(uint32_t r[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}
// 16 columns (one accumulator)
__device__ __forceinline__ void tc_ld16_issue(uint32_t taddr, uint32_t r[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tc_ld16_wait(uint32_t r[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 : "memory");
}
// 64 columns (four accumulators)
__device__ __forceinline__ void tc_ld64_issue(uint32_t taddr, uint32_t r[64]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tc_ld64_wait(uint32_t r[64]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]), "+r"(r[32]), "+r"(r[33]), "+r"(r[34]), "+r"(r[35]), "+r"(r[36]), "+r"(r[37]), "+r"(r[38]), "+r"(r[39]), "+r"(r[40]), "+r"(r[41]), "+r"(r[42]), "+r"(r[43]), "+r"(r[44]), "+r"(r[45]), "+r"(r[46]), "+r"(r[47]), "+r"(r[48]), "+r"(r[49]), "+r"(r[50]), "+r"(r[51]), "+r"(r[52]), "+r"(r[53]), "+r"(r[54]), "+r"(r[55]), "+r"(r[56]), "+r"(r[57]), "+r"(r[58]), "+r"(r[59]), "+r"(r[60]), "+r"(r[61]), "+r"(r[62]), "+r"(r[63])
                 :
                 : "memory");
}
template <int UNIT>
__device__ __forceinline__ void tc_ld_issue(uint32_t taddr, uint32_t* r) {
    if (UNIT == 4) tc_ld64_issue(taddr, r); else if (UNIT == 2) tc_ld32_issue(taddr, r); else tc_ld16_issue(taddr, r);
}
template <int UNIT>
__device__ __forceinline__ void tc_ld_wait(uint32_t* r) {
    if (UNIT == 4) tc_ld64_wait(r); else if (UNIT == 2) tc_ld32_wait(r); else tc_ld16_wait(r);
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle:
// groups of 8 rows are 1024 bytes apart (stride byte offset), the leading offset is unused.
__device__ __forceinline__ uint64_t tc_desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: D f32, A and B E4M3, both K-major, M = 128, N = 16.
constexpr uint32_t kTcIdesc = (1u << 4) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
// The barrier gets one arrival from this thread once all of its earlier cp.async copies have landed.
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(reinterpret_cast<uint64_t>(map)),
                 "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
// Bounded wait for a generation stamp written by another CTA of this launch.
__device__ __forceinline__ bool wait_stamp(const int* flag, int stamp, volatile int* abort_flag, uint64_t limit_ns) {
#pragma unroll 1
    for (int i = 0; i < 16; ++i) {  // the global timer is slow to read: only once the wait is clearly long
        if (ld_acquire(flag) == stamp) return true;
        __nanosleep(32);
    }
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t i = 0;; ++i) {
        if (ld_acquire(flag) == stamp) return true;
        __nanosleep(64);
        if ((i & 15) == 15) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > limit_ns) break;
        }
    }
    *abort_flag = 1;
    return false;
}

// Rendezvous of the finisher warps on an mbarrier, with the bounded wait of every other wait here:
// a thread that left because of an abort can never leave the others stuck in a barrier.
struct BoundedSync {
    uint64_t* bar;
    uint32_t phase;
    volatile int* abortp;
    uint64_t limit_ns;
    __device__ __forceinline__ bool sync() {
        mbar_arrive(bar);
        const bool ok = mbar_wait(bar, phase, abortp, limit_ns);
        phase ^= 1;
        return ok;
    }
};

// The four epilogue warps hold a finished row block: 128 output columns (one per thread) x the step's rows.
// Stages them as the next GEMV's activations: bf16 rounding, one amax/448 scale per row over the 128
// columns, E4M3 bytes (the arithmetic of the activation staging launch: glm53/gfx950/kernel.py:1440-1450).
__device__ __forceinline__ bool tc_stage_out(const mono_gemv_job& jb, int rows, int rb, int row_in_tile, int q, int lane, bool in_range,
                                             const float* total_acc, float (*s_amax)[kMaxRows], BoundedSync& es) {
    float v[kMaxRows];
#pragma unroll
    for (int c = 0; c < kMaxRows; ++c) {
        v[c] = bf16_round(total_acc[c]);
        const float am = warp_max(in_range ? fabsf(v[c]) : 0.f);
        if (lane == 0) s_amax[q][c] = am;
    }
    if (!es.sync()) return false;
#pragma unroll
    for (int c = 0; c < kMaxRows; ++c) {
        if (c < rows) {
            const float amax = fmaxf(fmaxf(s_amax[0][c], s_amax[1][c]), fmaxf(s_amax[2][c], s_amax[3][c]));
            uint8_t* dst = jb.stage_planes + (size_t)c * jb.stage_ld + rb * 128 + row_in_tile;
            float scale;
            if (jb.stage_fmt == MONO_ACT_A8) {
                scale = amax > 0.f ? amax / 448.f : 1.f;
                const float inv = amax > 0.f ? 448.f / amax : 1.f;
                if (in_range) *dst = f32_to_e4m3(v[c] * inv);
            } else {  // MONO_ACT_HILO: power-of-two scale, value = high byte + low byte
                const int code = code_ceil(fmaxf(amax, 7.888609052210118e-31f /* 2^-100 */) / 448.f);
                scale = exp2_code(code);
                const float sv = v[c] * exp2_code(254 - code);
                const uint8_t hb = f32_to_e4m3(sv);
                if (in_range) {
                    dst[0] = hb;
                    dst[jb.stage_plane_stride] = f32_to_e4m3(sv - e4m3_to_f32(hb));
                }
            }
            if (q == 0 && lane == 0) jb.stage_scale[(size_t)c * jb.stage_scale_ld + rb] = scale;
        }
    }
    return es.sync();  // the maxima may be overwritten by the next task
}

// The finisher warps (128 threads) learn that an up/gate task of `slot` is complete.  The CTA that counts
// the slot's last task turns the partial sums into the fed job's activations: sum over the K splits in
// order, SwiGLU, E4M3 with one amax/448 scale per 128 values (glm53/gfx950/kernel.py:1440-1450, :4352-5187).
// Every load of a (row, chunk) pair is issued before the first is used: under a saturated memory system a
// round trip costs microseconds, and the fed job waits for this.
__device__ __forceinline__ void tc_finish_up(const TcParams& p, const mono_gemv_job& jb, int slot, int tasks_per_slot,
                                             int stamp, int ft, volatile int* s_last, BoundedSync& fs) {
    const int fwarp = ft >> 5, lane = ft & 31;
    if (ft == 0) {
        __threadfence();  // the epilogue's stores (ordered before this by the mailbox barrier) before the count
        *s_last = (atomicAdd(jb.done + slot, 1) + 1 == tasks_per_slot) ? 1 : 0;
    }
    if (!fs.sync()) return;
    if (!*s_last) return;
    __threadfence();
    const mono_gemv_job& fed = p.a.job[jb.feeds_job - 1];
    const int inter = jb.n_rows >> 1, nchunks = inter >> 7, npairs = p.a.rows * nchunks;
    const float* base = jb.out + (size_t)(jb.mode == MONO_JOB_EXPERT_UP ? slot * jb.nsplit : 0) * jb.out_split_stride;
    uint8_t* planes = const_cast<uint8_t*>(fed.act) + (size_t)slot * fed.act_seg_stride;
    float* scales = const_cast<float*>(fed.ascale_f32) + (size_t)slot * fed.ascale_seg_stride;
    constexpr int kBatch = 2, kSplits = 4;  // pairs x K splits whose loads are in flight together
    for (int pair0 = fwarp * kBatch; pair0 < npairs; pair0 += 4 * kBatch) {
        float4 g4[kBatch], u4[kBatch];
#pragma unroll
        for (int q = 0; q < kBatch; ++q) g4[q] = u4[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < jb.nsplit; s0 += kSplits) {
            float4 x[kBatch][kSplits], y[kBatch][kSplits];
#pragma unroll
            for (int q = 0; q < kBatch; ++q) {
                const int pair = min(pair0 + q, npairs - 1);
                const int r = pair / nchunks, c = pair - r * nchunks;
                const float* gp = base + (size_t)r * jb.out_ld + c * 128 + 4 * lane;
#pragma unroll
                for (int s = 0; s < kSplits; ++s) {
                    const int ss = min(s0 + s, jb.nsplit - 1);
                    x[q][s] = __ldcg(reinterpret_cast<const float4*>(gp + (size_t)ss * jb.out_split_stride));
                    y[q][s] = __ldcg(reinterpret_cast<const float4*>(gp + (size_t)ss * jb.out_split_stride + inter));
                }
            }
#pragma unroll
            for (int q = 0; q < kBatch; ++q) {
#pragma unroll
                for (int s = 0; s < kSplits; ++s) {
                    if (s0 + s < jb.nsplit) {
                        g4[q].x += x[q][s].x; g4[q].y += x[q][s].y; g4[q].z += x[q][s].z; g4[q].w += x[q][s].w;
                        u4[q].x += y[q][s].x; u4[q].y += y[q][s].y; u4[q].z += y[q][s].z; u4[q].w += y[q][s].w;
                    }
                }
            }
        }
#pragma unroll
        for (int q = 0; q < kBatch; ++q) {
            const int pair = pair0 + q;
            if (pair >= npairs) break;
            const int r = pair / nchunks, c = pair - r * nchunks;
            const float gs[4] = {g4[q].x, g4[q].y, g4[q].z, g4[q].w}, us[4] = {u4[q].x, u4[q].y, u4[q].z, u4[q].w};
            float m[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) m[i] = gs[i] / (1.f + expf(-gs[i])) * us[i];
            const float amax = warp_max(fmaxf(fmaxf(fabsf(m[0]), fabsf(m[1])), fmaxf(fabsf(m[2]), fabsf(m[3]))));
            const float scale = amax > 0.f ? amax / 448.f : 1.f, inv = amax > 0.f ? 448.f / amax : 1.f;
            uint32_t w = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) w |= (uint32_t)f32_to_e4m3(m[i] * inv) << (8 * i);
            reinterpret_cast<uint32_t*>(planes + (size_t)r * fed.act_ld + c * 128)[lane] = w;
            if (lane == 0) scales[(size_t)r * fed.ascale_ld + c] = scale;
        }
    }
    fence_proxy_async();  // the fed job reads the planes with TMA
    __threadfence();
    if (!fs.sync()) return;
    if (ft == 0) {
        jb.done[slot] = 0;
        st_release(jb.ready + slot, stamp);
    }
}


template <int kTcUnit>
__global__ void __launch_bounds__(kTcThreads, 1) gemv_tc_kernel(const __grid_constant__ TcParams p) {
    constexpr int kTcMaxStages = tc_stages(kTcUnit), kTcTmemCols = tc_tmem_cols(kTcUnit), kTcScSlots = tc_sc_slots(kTcUnit);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    float* sc_ring = reinterpret_cast<float*>(smem + (size_t)kTcMaxStages * p.stage_bytes);  // [kTcScSlots][kTcScRows][32]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sc_ring + kTcScSlots * kTcScRows * kTcMaxSegTiles);
    uint64_t* full = bars;
    uint64_t* acc_full = full + kTcBarStages;
    uint64_t* acc_empty = acc_full + kTcBarStages;
    uint64_t* sc_full = acc_empty + kTcBarStages;
    uint64_t* sc_empty = sc_full + kTcScSlotsMax;
    uint64_t* mail_full = sc_empty + kTcScSlotsMax;  // epilogue -> finisher: an up/gate task's outputs are stored
    uint64_t* mail_free = mail_full + 2;
    uint64_t* fin_bar = mail_free + 2;
    uint64_t* epi_bar = fin_bar + 1;  // the four epilogue warps, when a job stages its output
    __shared__ int abort_flag, s_last[2];
    __shared__ float s_amax[4][kMaxRows];
    __shared__ uint32_t tmem_base_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // hot fields in registers: every inline asm with a memory clobber would make the compiler read them again
    const int rows = p.a.rows, stage_bytes = p.stage_bytes;
    if (tid == 0) {
        abort_flag = guard_failed(p.a.guard) ? 1 : 0;
        for (int i = 0; i < kTcMaxStages; ++i) mbar_init(&full[i], 1);
        for (int i = 0; i < kTcMaxStages; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
        for (int i = 0; i < kTcScSlots; ++i) { mbar_init(&sc_full[i], 32); mbar_init(&sc_empty[i], 4); }
        for (int i = 0; i < 2; ++i) { mbar_init(&mail_full[i], 128); mbar_init(&mail_free[i], 1); }
        mbar_init(fin_bar, 128);
        mbar_init(epi_bar, 128);
        mbar_fence_init();
    }
    if (warp == 1) tc_alloc(&tmem_base_s, kTcTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_launch_dependents();
    if (warp == 0) {
        // Weights do not depend on the kernel before this one: while it drains, pull this CTA's tiles towards
        // L2, up to kPrefetchTiles of them (the leading dense jobs only: their task list needs no upstream data).
        // Short projections then run out of L2 instead of paying the DRAM ramp after the wait.
        int budget = p.prefetch_tiles, base = 0;
        for (int j = 0; j < p.a.njobs && budget > 0; ++j) {
            const mono_gemv_job& jb = p.a.job[j];
            if (jb.mode != MONO_JOB_DENSE) break;
            const int nrb = tc_nrb(jb), ntask = nrb * jb.nsplit;
            const CUtensorMap* wmap = reinterpret_cast<const CUtensorMap*>(&jb.tmap);
            // this CTA's tasks of the job: global task index = base + local, taken round-robin over the grid
            int first = ((int)blockIdx.x - base) % (int)gridDim.x;
            if (first < 0) first += gridDim.x;
            for (int local = first; local < ntask && budget > 0; local += gridDim.x) {
                const TcSeg s = tc_make_seg(jb, local % nrb, local / nrb, 0);
                for (int t = lane; t < min(s.nt, budget); t += 32) tma_prefetch_3d(wmap, (s.t0 + t) * 128, s.row0, s.c2);
                if (lane == 0 && jb.wscale_f32) prefetch_l2(s.wsc);  // the segment's weight scales (at most 128 bytes)
                budget -= s.nt;
            }
            base += ntask;
        }
    }
    pdl_wait();
    MONO_TL(tl_gemv, 0);
    // chained jobs stamp their per-slot "activations ready" words with this launch's generation
    const int stamp = p.a.gen ? *reinterpret_cast<const volatile int*>(p.a.gen) + 1 : 1;

    int cnt[MONO_GEMV_MAX_JOBS], nexp[MONO_GEMV_MAX_JOBS], total = 0;
#pragma unroll
    for (int j = 0; j < MONO_GEMV_MAX_JOBS; ++j) {
        cnt[j] = 0;
        nexp[j] = 0;
        if (j < p.a.njobs) {
            const mono_gemv_job& jb = p.a.job[j];
            const int nrb = tc_nrb(jb);
            if (jb.mode == MONO_JOB_DENSE) {
                cnt[j] = nrb * jb.nsplit;
            } else {
                nexp[j] = min(*jb.n_expert, jb.max_expert);
                cnt[j] = (jb.mode == MONO_JOB_EXPERT_UP) ? nexp[j] * nrb * jb.nsplit : nrb * jb.nsplit;
            }
        }
        total += cnt[j];
    }
    // the step's expert lists in shared memory: a global load per segment would put an L2 round trip on
    // every role's path (a down segment is only two tiles long)
    __shared__ int s_elist[MONO_GEMV_MAX_JOBS][kTcListCache];
    for (int j = 0; j < p.a.njobs; ++j)
        if (p.a.job[j].mode != MONO_JOB_DENSE)
            for (int i = tid; i < min(nexp[j], kTcListCache); i += kTcThreads) s_elist[j][i] = p.a.job[j].expert_list[i];
    __syncthreads();
    volatile int* abortp = &abort_flag;
    const uint64_t wait_ns = p.a.wait_ns ? p.a.wait_ns : kWaitLimitNs;

// every role walks the same (task, segment, tile) sequence
#define TC_FOR_EACH_SEGMENT(...)                                                                                \
    for (int task = blockIdx.x; task < total && !*abortp; task += gridDim.x) {                                  \
        int j = 0, local = task;                                                                                \
        while (local >= cnt[j]) { local -= cnt[j]; ++j; }                                                       \
        const mono_gemv_job& jb = p.a.job[j];                                                                   \
        const int planes = jb.planes;                                                                           \
        (void)planes;                                                                                           \
        const int nrb = tc_nrb(jb);                                                                             \
        int u = 0, nseg = 1;                                                                                    \
        if (jb.mode == MONO_JOB_EXPERT_UP) { u = local / (nrb * jb.nsplit); local -= u * nrb * jb.nsplit; }     \
        const int u_up = u, rb = local % nrb, ks = local / nrb;                                                 \
        if (jb.mode == MONO_JOB_EXPERT_DOWN) nseg = (nexp[j] > ks) ? (nexp[j] - ks + jb.nsplit - 1) / jb.nsplit : 0; \
        (void)u_up; (void)rb;                                                                                   \
        TASK_BEGIN                                                                                              \
        for (int sgi = 0; sgi < nseg && !*abortp; ++sgi) {                                                      \
            if (jb.mode == MONO_JOB_EXPERT_DOWN) u = ks + sgi * jb.nsplit;                                      \
            const TcSeg s = tc_make_seg(jb, rb, ks, u, s_elist[j]);                                             \
            __VA_ARGS__                                                                                         \
        }                                                                                                       \
        TASK_END                                                                                                \
    }

    if (warp == 0) {
        // ------------------------------------------------------------ producer: scales by cp.async, tiles by TMA
        int stage = 0, slot = 0;
        uint32_t phase = 0, sphase = 0, ready_mask = 0;
#ifdef MONO_TIMELINE
        int tl_seg = 0;
#endif
#define TASK_BEGIN
#define TASK_END
        TC_FOR_EACH_SEGMENT({
            // the segment's scales: rows 0..15 activation scales [nt], row 16 weight scales, row 17 coefficients
            int ok = 1;
            if (jb.ready && jb.feeds_job == 0) {
                // a fed job: the activations of a slot come from an up/gate job of this launch.  One round of
                // flag loads per task (lane s looks at segment s); only segments that were not ready then
                // are polled again when their turn comes.
                const bool down = jb.mode == MONO_JOB_EXPERT_DOWN;
                if (sgi == 0) {
                    const bool r = lane < nseg ? ld_acquire(jb.ready + (down ? ks + lane * jb.nsplit : 0)) == stamp : true;
                    ready_mask = __ballot_sync(0xffffffffu, r);
                    if (ready_mask != 0xffffffffu && lane == 0) {
                        // pull the whole task's weight tiles towards L2 while the up/gate jobs finish
                        const CUtensorMap* wmap = reinterpret_cast<const CUtensorMap*>(&jb.tmap);
                        for (int sg2 = 0; sg2 < nseg; ++sg2) {
                            const TcSeg s2 = tc_make_seg(jb, rb, ks, down ? ks + sg2 * jb.nsplit : u, s_elist[j]);
                            for (int t = 0; t < s2.nt; ++t) tma_prefetch_3d(wmap, (s2.t0 + t) * 128, s2.row0, s2.c2);
                        }
                    }
                }
                if (sgi >= 32 || !((ready_mask >> sgi) & 1u)) {
                    if (lane == 0) {
                        ok = wait_stamp(jb.ready + (down ? u : 0), stamp, abortp, wait_ns) ? 1 : 0;
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                }
                // (the writer ordered its stores against the async proxy before it released the stamp)
            }
#ifdef MONO_TIMELINE
#ifndef MONO_TLP_FIRST
#define MONO_TLP_FIRST 4  // the first of the three segments whose producer steps are stamped
#endif
#define TLP(k) do { if (blockIdx.x == 0 && lane == 0 && tl_seg >= MONO_TLP_FIRST && tl_seg < MONO_TLP_FIRST + 3) tl_gemv[153][(tl_seg - MONO_TLP_FIRST) * 5 + (k)] = globaltimer_ns(); } while (0)
#else
#define TLP(k) do { } while (0)
#endif
            TLP(0);
            if (lane == 0) ok = mbar_wait(&sc_empty[slot], sphase ^ 1, abortp, wait_ns) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            TLP(1);
            float* sl = sc_ring + (size_t)slot * kTcScRows * kTcMaxSegTiles;
            for (int i = lane; i < rows * s.nt; i += 32) {
                const int c = i / s.nt, t = i - c * s.nt;
                cp_async4(&sl[c * kTcMaxSegTiles + t], s.asc + (size_t)c * jb.ascale_ld + t);
            }
            if (lane < s.nt) cp_async4(&sl[16 * kTcMaxSegTiles + lane], s.wsc + lane);
            if (s.coef && lane < rows) cp_async4(&sl[17 * kTcMaxSegTiles + lane], s.coef + lane);
            cp_async_arrive(&sc_full[slot]);
            if (++slot == kTcScSlots) { slot = 0; sphase ^= 1; }
            TLP(2);
            if (lane == 0) {
                const CUtensorMap* wmap = reinterpret_cast<const CUtensorMap*>(&jb.tmap);
                const CUtensorMap* amap = reinterpret_cast<const CUtensorMap*>(&jb.act_tmap);
                for (int t = 0; t < s.nt; t += kTcUnit) {
                    const int n2 = min(kTcUnit, s.nt - t);
                    if (!mbar_wait(&acc_full[stage], phase ^ 1, abortp, wait_ns)) break;  // the MMAs of the stage's last unit are done
                    TLP(3);
                    uint8_t* st = ring + (size_t)stage * stage_bytes;
                    mbar_expect_tx(&full[stage], n2 * (kTcABytes + planes * kTcBBytes));
                    for (int i = 0; i < n2; ++i) {
                        tma_load_3d(st + i * kTcABytes, wmap, (s.t0 + t + i) * 128, s.row0, s.c2, &full[stage]);
                        for (int pl = 0; pl < planes; ++pl)
                            tma_load_3d(st + kTcUnit * kTcABytes + (i * planes + pl) * kTcBBytes, amap, (s.t0 + t + i) * 128, 0,
                                        s.aset * planes + pl, &full[stage]);
                    }
                    if (++stage == kTcMaxStages) { stage = 0; phase ^= 1; }
                }
                TLP(4);
#ifdef MONO_TIMELINE
                if (blockIdx.x == 0 && tl_seg < MONO_TL_POINTS) tl_gemv[150][tl_seg] = globaltimer_ns();
#endif
            }
#ifdef MONO_TIMELINE
            ++tl_seg;
#endif
            __syncwarp();
        })
#undef TASK_BEGIN
#undef TASK_END
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0, g = 0;
#ifdef MONO_TIMELINE
            int tl_seg = 0;
#endif
#define TASK_BEGIN
#define TASK_END
            TC_FOR_EACH_SEGMENT({
                for (int t = 0; t < s.nt; t += kTcUnit) {
                    const int n2 = min(kTcUnit, s.nt - t);
                    if (!mbar_wait(&full[stage], phase, abortp, wait_ns)) break;
                    if (!mbar_wait(&acc_empty[stage], phase ^ 1, abortp, wait_ns)) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(ring + (size_t)stage * stage_bytes);
                    for (int i = 0; i < n2; ++i) {
                        const uint64_t adesc = tc_desc_sw128(sa + i * kTcABytes);
                        uint32_t accumulate = 0;
                        for (int pl = 0; pl < planes; ++pl) {
                            const uint64_t bdesc = tc_desc_sw128(sa + kTcUnit * kTcABytes + (i * planes + pl) * kTcBBytes);
#pragma unroll
                            for (int k = 0; k < 4; ++k) {  // 32 bytes of K per MMA: the start address moves by 32 B
                                tc_mma_f8(tmem_base + stage * (16 * kTcUnit) + i * 16, adesc + 2 * k, bdesc + 2 * k, kTcIdesc, accumulate);
                                accumulate = 1;
                            }
                        }
                    }
                    // one commit serves both: the accumulators are complete (epilogue) and the stage's shared
                    // memory has been read (producer); stage s and accumulator pair s always go together
                    tc_commit(&acc_full[stage]);
                    g += n2;
                    if (++stage == kTcMaxStages) { stage = 0; phase ^= 1; }
                }
#ifdef MONO_TIMELINE
                if (blockIdx.x == 0 && tl_seg < MONO_TL_POINTS) tl_gemv[151][tl_seg] = globaltimer_ns();
                ++tl_seg;
#endif
            })
#undef TASK_BEGIN
#undef TASK_END
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue (TMEM lanes 32 * (warp % 4) ..)
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        uint32_t g = 0, sphase = 0;
        int slot = 0;
        uint32_t nfeed = 0;
        const uint32_t tmem_lane = tmem_base + ((uint32_t)(q * 32) << 16);
        uint32_t dn[16 * kTcUnit];  // raw registers of the accumulator load in flight
        int stage = 0;
        uint32_t phase = 0;
        bool have_next = false;
        BoundedSync es{epi_bar, 0u, abortp, wait_ns};
        float total_acc[kMaxRows];
        int tl_n = 1;  // timeline: the end of this CTA's n-th task (first epilogue warp's lane 0)
        (void)tl_n;
#ifdef MONO_TIMELINE
        int tl_seg = 0;
#endif
#define TASK_BEGIN \
        _Pragma("unroll") for (int c = 0; c < kMaxRows; ++c) total_acc[c] = 0.f;
#define TASK_END                                                                                              \
        if (!*abortp) {                                                                                       \
            const int out_row = rb * 128 + row_in_tile;                                                       \
            const int row_in_mat = (jb.mode == MONO_JOB_DENSE && jb.rb_per_mat > 0) ? (rb % jb.rb_per_mat) * 128 + row_in_tile : out_row; \
            float* out = jb.out + (size_t)((jb.mode == MONO_JOB_EXPERT_UP ? u_up * jb.nsplit : 0) + ks) * jb.out_split_stride; \
            if (row_in_mat < jb.n_rows) {                                                                     \
                _Pragma("unroll") for (int c = 0; c < kMaxRows; ++c)                                          \
                    if (c < rows) out[(size_t)c * jb.out_ld + out_row] = total_acc[c];                    \
            }                                                                                                 \
            if (jb.stage_planes) tc_stage_out(jb, rows, rb, row_in_tile, q, lane, row_in_mat < jb.n_rows, total_acc, s_amax, es); \
            if (jb.feeds_job > 0) {                                                                           \
                const uint32_t k = nfeed & 1;                                                                 \
                if (mbar_wait(&mail_free[k], ((nfeed >> 1) & 1) ^ 1, abortp, wait_ns)) mbar_arrive(&mail_full[k]);     \
                ++nfeed;                                                                                      \
            }                                                                                                 \
            if (warp == 2 && lane == 0) { MONO_TL_AT(tl_gemv, tl_n); ++tl_n; }                                \
        }
        TC_FOR_EACH_SEGMENT({
            if (!mbar_wait(&sc_full[slot], sphase, abortp, wait_ns)) break;
            const float* sl = sc_ring + (size_t)slot * kTcScRows * kTcMaxSegTiles;
            float seg_acc[kMaxRows];
#pragma unroll
            for (int c = 0; c < kMaxRows; ++c) seg_acc[c] = 0.f;
            for (int t = 0; t < s.nt; t += kTcUnit) {
                const int n2 = min(kTcUnit, s.nt - t);
                if (!have_next) {
                    if (!mbar_wait(&acc_full[stage], phase, abortp, wait_ns)) break;
                    tc_fence_after();
                    tc_ld_issue<kTcUnit>(tmem_lane + stage * (16 * kTcUnit), dn);
                }
                tc_ld_wait<kTcUnit>(dn);
                float d[16 * kTcUnit];
#pragma unroll
                for (int c = 0; c < 16 * kTcUnit; ++c) d[c] = __uint_as_float(dn[c]);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[stage]);
                if (++stage == kTcMaxStages) { stage = 0; phase ^= 1; }
                {
                    // if the next unit is complete already, start its load before the math on this one
                    int h = lane == 0 ? (mbar_try_wait(&acc_full[stage], phase) ? 1 : 0) : 0;
                    have_next = __shfl_sync(0xffffffffu, h, 0) != 0;
                    if (have_next) {
                        tc_fence_after();
                        tc_ld_issue<kTcUnit>(tmem_lane + stage * (16 * kTcUnit), dn);
                    }
                }
#pragma unroll
                for (int i = 0; i < kTcUnit; ++i) {
                    if (i < n2) {
                        const float ws = sl[16 * kTcMaxSegTiles + t + i];
#pragma unroll
                        for (int c = 0; c < kMaxRows; ++c)
                            if (c < rows) seg_acc[c] += d[i * 16 + c] * (ws * sl[c * kTcMaxSegTiles + t + i]);
                    }
                }
                g += n2;
            }
#pragma unroll
            for (int c = 0; c < kMaxRows; ++c)
                if (c < rows) total_acc[c] += seg_acc[c] * (s.coef ? sl[17 * kTcMaxSegTiles + c] : 1.f);
            __syncwarp();
            if (lane == 0) mbar_arrive(&sc_empty[slot]);
            if (++slot == kTcScSlots) { slot = 0; sphase ^= 1; }
#ifdef MONO_TIMELINE
            if (blockIdx.x == 0 && warp == 2 && lane == 0 && tl_seg < MONO_TL_POINTS) tl_gemv[152][tl_seg] = globaltimer_ns();
            ++tl_seg;
#endif
        })
#undef TASK_BEGIN
#undef TASK_END
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");  // nothing in flight when TMEM goes (abort paths)
    }
    if (warp >= 6) {
        const int ft = tid - 192;
        BoundedSync fs{fin_bar, 0u, abortp, wait_ns};
        // ------------------------------------------------------------ finisher: counts finished up/gate tasks
        uint32_t nfeed = 0;
#define TASK_BEGIN
#define TASK_END                                                                                              \
        if (jb.feeds_job > 0 && !*abortp) {                                                                   \
            const uint32_t k = nfeed & 1;                                                                     \
            if (mbar_wait(&mail_full[k], (nfeed >> 1) & 1, abortp, wait_ns)) {                                         \
                tc_finish_up(p, jb, jb.mode == MONO_JOB_EXPERT_UP ? u_up : 0, nrb * jb.nsplit, stamp, ft, &s_last[k], fs); \
                if (ft == 0) mbar_arrive(&mail_free[k]);                                                    \
            }                                                                                                 \
            ++nfeed;                                                                                          \
        }
        TC_FOR_EACH_SEGMENT({ (void)s; })
#undef TASK_BEGIN
#undef TASK_END
    }
#undef TC_FOR_EACH_SEGMENT
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before the CTA's memory goes
        if (tid == 0 && !guard_failed(p.a.guard)) guard_fail(p.a.guard, MONO_ERR_DEADLINE, 101);
    }
    if (warp == 1) {
        tc_fence_after();
        tc_dealloc(tmem_base, kTcTmemCols);
    }
    if (tid == 0 && p.a.gen) {
        // the last CTA to leave starts the next generation
        __threadfence();
        if (atomicAdd(p.a.gen + 1, 1) == (int)gridDim.x - 1) {
            p.a.gen[1] = 0;
            if (guard_failed(p.a.guard)) {
                // a launch that gave up leaves partial task counts behind: every other CTA has left, so
                // the counters can go back to zero for the launch after the host clears the guard
                for (int j = 0; j < p.a.njobs; ++j) {
                    const mono_gemv_job& jb = p.a.job[j];
                    if (jb.feeds_job > 0 && jb.done)
                        for (int i = 0; i < (jb.mode == MONO_JOB_EXPERT_UP ? jb.max_expert : 1); ++i) jb.done[i] = 0;
                }
            }
            __threadfence();
            atomicAdd(p.a.gen, 1);
        }
    }
}

}  // namespace mono

static int g_mono_gemv_tc = 1;
extern "C" int mono_set_gemv_tcgen05(int on) {
    const int old = g_mono_gemv_tc;
    g_mono_gemv_tc = on ? 1 : 0;
    return old;
}
int mono_gemv_tc_enabled() { return g_mono_gemv_tc; }

// Picks the pipeline unit and the shared-memory size of a validated FP8 argument block.
static int tc_plan(const mono_gemv_args* a, mono::TcParams* pp, int* unit_out, size_t* smem_out) {
    using namespace mono;
    TcParams& p = *pp;
    p.a = *a;
    int planes = 1;
    for (int j = 0; j < a->njobs; ++j) planes = a->job[j].planes > planes ? a->job[j].planes : planes;
    // as many stages as fit: the bytes in flight per SM are what hides the DRAM latency
    const int kSmemMax = 224 * 1024;  // 227 KB less the static part (expert lists, flags)
    // two-tile pipeline units pay off when a CTA streams many tiles (expert jobs, large dense matrices: 735 vs
    // 895 us per config-3 layer at TP 1); short dense launches are quicker with one-tile units and more stages
    static const int forced_unit = [] { const char* e = getenv("MONO_TC_UNIT"); return e ? (e[0] == '4' ? 4 : e[0] == '2' ? 2 : 1) : 0; }();
    // (four-tile units: 710 us, the up/gate launch at 0.90 of the measured copy bandwidth; they need long K
    // runs per segment, or a stage is mostly empty)
    static const long tile_floor = [] { const char* e = getenv("MONO_TC_UNIT2_TILES"); return e ? atol(e) : 12L; }();
    long dense_tiles = 0;
    bool expert = false;
    int min_seg = 1 << 30;
    for (int j = 0; j < a->njobs; ++j) {
        const mono_gemv_job& jb = a->job[j];
        if (jb.mode != MONO_JOB_DENSE) {
            expert = true;
            const int seg = jb.mode == MONO_JOB_EXPERT_DOWN ? jb.k_tiles : (jb.split_tiles < jb.k_tiles ? jb.split_tiles : jb.k_tiles);
            min_seg = seg < min_seg ? seg : min_seg;
        } else {
            dense_tiles += (long)(jb.rb_per_mat > 0 ? jb.n_mats * jb.rb_per_mat : (jb.n_rows + 127) / 128) * jb.k_tiles;
        }
    }
    int unit = forced_unit ? forced_unit : (expert && min_seg >= 8) ? 4 : (expert || dense_tiles >= tile_floor * mono_sm_count()) ? 2 : 1;
    if (unit == 4 && planes != 1) unit = 2;  // four-tile stages fit with one activation plane only
    const size_t fixed = 1024 + (size_t)tc_sc_slots(unit) * kTcScRows * kTcMaxSegTiles * sizeof(float) + 512;
    // MONO_TC_PREFETCH_TILES: 24 tiles = 384 KB per CTA, 57 MB over the grid
    static const int prefetch_tiles = [] { const char* e = getenv("MONO_TC_PREFETCH_TILES"); return e ? atoi(e) : 24; }();
    p.prefetch_tiles = prefetch_tiles;
    p.stage_bytes = unit * (kTcABytes + planes * kTcBBytes);
    p.stages = (int)((kSmemMax - fixed) / p.stage_bytes);
    if (p.stages < tc_stages(unit)) return MONO_E_ARG;
    p.stages = tc_stages(unit);  // stage s feeds accumulator set s
    const size_t smem = fixed + (size_t)p.stages * p.stage_bytes;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        cudaError_t e = cudaFuncSetAttribute(gemv_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_tc_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        if (e != cudaSuccess) return (int)e;
        mono::attr_done(attr_once);
    }
    *unit_out = unit;
    *smem_out = smem;
    return 0;
}

// CTAs of this launch's kernel that the device keeps resident at once (occupancy x SM count).
static int tc_resident(int unit, size_t smem) {
    using namespace mono;
    // the answer depends on (device, unit, shared memory): asked once each, outside any hot path
    struct Entry { int dev, unit; size_t smem; int resident; };
    static std::mutex mu;
    static std::vector<Entry> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    {
        std::lock_guard<std::mutex> lk(mu);
        for (const Entry& en : cache)
            if (en.dev == dev && en.unit == unit && en.smem == smem) return en.resident;
    }
    int per_sm = 0;
    cudaError_t e = unit == 4   ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_tc_kernel<4>, kTcThreads, smem)
                    : unit == 2 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_tc_kernel<2>, kTcThreads, smem)
                                : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_tc_kernel<1>, kTcThreads, smem);
    if (e != cudaSuccess) return -1;
    const int sms = mono_sm_count();
    const int resident = sms > 0 ? per_sm * sms : -1;
    if (resident > 0) {
        std::lock_guard<std::mutex> lk(mu);
        cache.push_back({dev, unit, smem, resident});
    }
    return resident;
}

// Launches the tcgen05 kernel for an FP8 argument block that mono_gemv_launch has validated.
int mono_gemv_tc_launch(const mono_gemv_args* a, long tasks, cudaStream_t st) {
    using namespace mono;
    for (int j = 0; j < a->njobs; ++j) {
        const mono_gemv_job& jb = a->job[j];
        const int seg = jb.mode == MONO_JOB_EXPERT_DOWN ? jb.k_tiles : (jb.split_tiles < jb.k_tiles ? jb.split_tiles : jb.k_tiles);
        if (seg > kTcMaxSegTiles) {
            mono_set_error("mono_gemv_launch: job %d: a segment may span at most %d tiles", j, kTcMaxSegTiles);
            return MONO_E_ARG;
        }
        if (jb.stage_planes) {
            if (jb.mode != MONO_JOB_DENSE || jb.nsplit != 1 || jb.feeds_job > 0 || !jb.stage_scale || jb.stage_ld < 128 || jb.stage_scale_ld < 1 ||
                (jb.stage_fmt != MONO_ACT_A8 && jb.stage_fmt != MONO_ACT_HILO) || (jb.stage_fmt == MONO_ACT_HILO && jb.stage_plane_stride <= 0)) {
                mono_set_error("mono_gemv_launch: job %d: only a dense job without K splits can stage its output "
                               "(stage_planes, stage_scale, their leading dimensions and stage_fmt A8 or HILO required)", j);
                return MONO_E_ARG;
            }
        }
        if (jb.feeds_job > 0) {
            const int f = jb.feeds_job - 1;
            const bool shape_ok = jb.mode != MONO_JOB_EXPERT_DOWN && jb.rb_per_mat == 0 && (jb.n_rows & 255) == 0;
            if (!a->gen || !jb.done || !jb.ready || f <= j || f >= a->njobs || !shape_ok || a->job[f].ready != jb.ready ||
                a->job[f].planes != 1 || a->job[f].k_tiles * 128 != jb.n_rows / 2 ||
                (jb.mode == MONO_JOB_EXPERT_UP) != (a->job[f].mode == MONO_JOB_EXPERT_DOWN)) {
                mono_set_error("mono_gemv_launch: job %d: a chained up/gate job needs gen, done, ready, 2 * inter rows with "
                               "inter a multiple of 128, and a later job of matching kind with one E4M3 plane of inter bytes", j);
                return MONO_E_ARG;
            }
        }
    }
    TcParams p;
    int unit = 1;
    size_t smem = 0;
    if (int rc = tc_plan(a, &p, &unit, &smem)) return rc;
    int grid = a->max_ctas > 0 ? a->max_ctas : mono_sm_count();
    if (grid > tasks) grid = (int)tasks;
    if (grid < 1) grid = 1;
    bool chained = false;
    for (int j = 0; j < a->njobs; ++j) chained = chained || a->job[j].feeds_job > 0;
    if (chained) {
        // CTAs of a chained launch wait on stamps that other CTAs of the same launch write: every CTA
        // has to be resident (minimax_m31/runner.py:125-143 refuses a grid above the co-resident count)
        const int resident = tc_resident(unit, smem);
        if (resident < 1 || grid > resident) {
            mono_set_error("mono_gemv_launch: a chained launch of %d CTAs exceeds the %d the device keeps resident", grid, resident);
            return MONO_E_ARG;
        }
    }
    cudaError_t e = unit == 4   ? launch_k(gemv_tc_kernel<4>, grid, kTcThreads, smem, st, p)
                    : unit == 2 ? launch_k(gemv_tc_kernel<2>, grid, kTcThreads, smem, st, p)
                                : launch_k(gemv_tc_kernel<1>, grid, kTcThreads, smem, st, p);
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

// CTAs the device keeps resident for this argument block's kernel (the tcgen05 FP8 kernel; other
// weight kinds run one CTA per SM).  A chained launch needs its whole grid resident.
extern "C" int mono_gemv_max_resident_ctas(const mono_gemv_args* a) {
    if (!a || a->njobs < 1 || a->njobs > MONO_GEMV_MAX_JOBS) {
        mono_set_error("mono_gemv_max_resident_ctas: njobs in 1..%d required", MONO_GEMV_MAX_JOBS);
        return MONO_E_ARG;
    }
    if (a->wkind != MONO_W_FP8 || !g_mono_gemv_tc) return mono_sm_count();
    mono::TcParams p;
    int unit = 1;
    size_t smem = 0;
    if (int rc = tc_plan(a, &p, &unit, &smem)) return rc > 0 ? -rc : rc;
    return tc_resident(unit, smem);
}

#ifdef MONO_TIMELINE
// Copies the tcgen05 GEMV's stamps of the last launch to `out` (MONO_TL_CTAS x MONO_TL_POINTS); blocks the host.
extern "C" int mono_timeline_read_gemv_tc(unsigned long long* out, int* ctas, int* points) {
    *ctas = MONO_TL_CTAS;
    *points = MONO_TL_POINTS;
    return (int)cudaMemcpyFromSymbol(out, mono::tl_gemv, sizeof(unsigned long long) * MONO_TL_CTAS * MONO_TL_POINTS);
}
#endif
