// MXFP4 weight-streaming GEMV on tcgen05: E2M1 weights x E4M3 activations (kind::f8f6f4), one MMA per
// 32-value scale group, each group in its own TMEM accumulator; the epilogue applies the two E8M0 codes
// of the group (weight row x group, activation row x group) and adds in f32.
//
// Same contract and task list as gemv.cu's MXFP4 consumer (reference: minimax_m31/a16w8.py and the MXFP4
// expert stages of glm53_flash/gfx950/kernel.py:4025-4392; E8M0 rule common/mx.py:27-39).  TMA reads the
// packed nibbles in place (128 elements = 64 bytes of a row per box) and writes them to shared memory in
// the padded layout the MMA reads 4-bit operands in (16 elements per 16 bytes, 128-byte rows, 128-byte
// swizzle).  Activations are MONO_ACT_MX8N planes (natural k order) read through their own descriptor.
//
// 192 threads: warp 0 TMA + scales (cp.async into a 2-slot ring), one thread of warp 1 issues the MMAs,
// warps 2..5 own the 128 TMEM lanes.  Every wait is bounded; TMEM is freed on every exit path.
#include "mono_common.cuh"

extern void mono_set_error(const char* fmt, ...);

namespace mono {
namespace tc4 {

constexpr int kThreads = 192;
constexpr int kUnit = 2;                // k tiles (128 elements) per stage: one barrier round trip and one commit for both
constexpr int kStages = 4;              // a stage = kUnit tiles: 16 KB of padded weights + 2 KB of activations each
constexpr int kABytes = 128 * 128;      // padded: 128 rows x 128 bytes hold 128 x 128 nibbles
constexpr int kBBytes = 16 * 128;
constexpr int kStageBytes = kUnit * (kABytes + kBBytes);
constexpr int kTxBytes = kABytes / 2 + kBBytes;  // per tile: the barrier counts the packed nibbles TMA fetched, not the padded rows it wrote
constexpr int kTmemCols = 512;          // kStages x kUnit tiles x 4 groups x 16 columns
constexpr int kMaxSegTiles = 16;        // k tiles (128 elements) per segment
constexpr int kScSlots = 2;
constexpr int kSlotWords = kMaxSegTiles * 128 + kMaxSegTiles * 16 + 16;  // weight codes, activation codes, coefficients

struct Params {
    mono_gemv_args a;
};

struct Seg {
    int c2, row0, t0, nt, aset;  // t0, nt in 128-element tiles
    const uint8_t* asc;
    const uint8_t* wsc;
    const float* coef;
};

__device__ __forceinline__ int nrb_of(const mono_gemv_job& j) { return (j.n_rows + 127) >> 7; }

__device__ __forceinline__ Seg make_seg(const mono_gemv_job& j, int rb, int ks, int u, const int* elist) {
    Seg s;
    int mat = 0;
    // K in 128-element tiles: exact when the caller gave it (a K that ends inside a 128-byte tile of nibbles)
    const int total4 = j.k_tiles4 > 0 ? j.k_tiles4 : 2 * j.k_tiles;
    if (j.mode == MONO_JOB_DENSE) {
        s.t0 = 2 * ks * j.split_tiles;
        s.nt = min(2 * j.split_tiles, total4 - s.t0);
        s.aset = 0;
        s.coef = nullptr;
    } else if (j.mode == MONO_JOB_EXPERT_UP) {
        mat = (u < 128) ? elist[u] : j.expert_list[u];
        s.t0 = 2 * ks * j.split_tiles;
        s.nt = min(2 * j.split_tiles, total4 - s.t0);
        s.aset = 0;
        s.coef = nullptr;
    } else {
        mat = (u < 128) ? elist[u] : j.expert_list[u];
        s.t0 = 0;
        s.nt = total4;
        s.aset = u;
        s.coef = j.coef ? j.coef + (size_t)u * kMaxRows : nullptr;
    }
    s.c2 = mat;
    s.row0 = j.row_off + rb * 128;
    s.asc = j.ascale_e8 + (size_t)s.aset * j.ascale_seg_stride + (size_t)s.t0 * 4;
    s.wsc = j.wscale_e8 + (size_t)mat * j.wscale_mat_stride + (size_t)s.row0 * j.wscale_ld + (size_t)s.t0 * 4;
    return s;
}

// ---- tcgen05 wrappers (local to this file)
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mma_f8f6f4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    // a fresh accumulator per MMA: the predicate (accumulate) is always false
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc)
        : "memory");
}
// 64 TMEM columns (the four group accumulators of a tile) of this thread's lane
__device__ __forceinline__ void ld64(uint32_t taddr, uint32_t r[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
          "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]),
          "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]),
          "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// K-major tile with 128-byte rows and the 128-byte swizzle: groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// D f32, A E2M1 (format 5), B E4M3 (format 0), both K-major, M = 128, N = 16
constexpr uint32_t kIdesc = (1u << 4) | (5u << 7) | (0u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void cp4(void* dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 2^(cw + ca - 254): the product of two E8M0 scales as an f32 (underflow to zero)
__device__ __forceinline__ float e8_product(uint32_t cw, uint32_t ca) {
    const int e = (int)cw + (int)ca - 127;
    return __uint_as_float((uint32_t)max(e, 0) << 23);
}

__global__ void __launch_bounds__(kThreads, 1) gemv_tc4_kernel(const __grid_constant__ Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    uint32_t* sc_ring = reinterpret_cast<uint32_t*>(smem + (size_t)kStages * kStageBytes);
    float* asf_all = reinterpret_cast<float*>(sc_ring + kScSlots * kSlotWords);  // [4 epilogue warps][tile][16 rows][4 groups]
    uint64_t* bars = reinterpret_cast<uint64_t*>(asf_all + 4 * kMaxSegTiles * 64);
    uint64_t* full = bars;
    uint64_t* acc_full = full + kStages;
    uint64_t* acc_empty = acc_full + kStages;
    uint64_t* sc_full = acc_empty + kStages;
    uint64_t* sc_empty = sc_full + kScSlots;
    __shared__ int abort_flag;
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_elist[MONO_GEMV_MAX_JOBS][128];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rows = p.a.rows;
    if (tid == 0) {
        abort_flag = guard_failed(p.a.guard) ? 1 : 0;
        for (int i = 0; i < kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
        for (int i = 0; i < kScSlots; ++i) { mbar_init(&sc_full[i], 32); mbar_init(&sc_empty[i], 4); }
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&tmem_base_s, kTmemCols);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_launch_dependents();
    pdl_wait();

    int cnt[MONO_GEMV_MAX_JOBS], nexp[MONO_GEMV_MAX_JOBS], total = 0;
#pragma unroll
    for (int j = 0; j < MONO_GEMV_MAX_JOBS; ++j) {
        cnt[j] = 0;
        nexp[j] = 0;
        if (j < p.a.njobs) {
            const mono_gemv_job& jb = p.a.job[j];
            const int nrb = nrb_of(jb);
            if (jb.mode == MONO_JOB_DENSE) {
                cnt[j] = nrb * jb.nsplit;
            } else {
                nexp[j] = min(*jb.n_expert, jb.max_expert);
                cnt[j] = (jb.mode == MONO_JOB_EXPERT_UP) ? nexp[j] * nrb * jb.nsplit : nrb * jb.nsplit;
            }
        }
        total += cnt[j];
    }
    for (int j = 0; j < p.a.njobs; ++j)
        if (p.a.job[j].mode != MONO_JOB_DENSE)
            for (int i = tid; i < min(nexp[j], 128); i += kThreads) s_elist[j][i] = p.a.job[j].expert_list[i];
    __syncthreads();
    volatile int* abortp = &abort_flag;
    const uint64_t wait_ns = p.a.wait_ns ? p.a.wait_ns : kWaitLimitNs;

#define T4_FOR_EACH_SEGMENT(...)                                                                                \
    for (int task = blockIdx.x; task < total && !*abortp; task += gridDim.x) {                                  \
        int j = 0, local = task;                                                                                \
        while (local >= cnt[j]) { local -= cnt[j]; ++j; }                                                       \
        const mono_gemv_job& jb = p.a.job[j];                                                                   \
        const int nrb = nrb_of(jb);                                                                             \
        int u = 0, nseg = 1;                                                                                    \
        if (jb.mode == MONO_JOB_EXPERT_UP) { u = local / (nrb * jb.nsplit); local -= u * nrb * jb.nsplit; }     \
        const int u_up = u, rb = local % nrb, ks = local / nrb;                                                 \
        if (jb.mode == MONO_JOB_EXPERT_DOWN) nseg = (nexp[j] > ks) ? (nexp[j] - ks + jb.nsplit - 1) / jb.nsplit : 0; \
        (void)u_up; (void)rb;                                                                                   \
        TASK_BEGIN                                                                                              \
        for (int sgi = 0; sgi < nseg && !*abortp; ++sgi) {                                                      \
            if (jb.mode == MONO_JOB_EXPERT_DOWN) u = ks + sgi * jb.nsplit;                                      \
            const Seg s = make_seg(jb, rb, ks, u, s_elist[j]);                                                  \
            __VA_ARGS__                                                                                         \
        }                                                                                                       \
        TASK_END                                                                                                \
    }

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        int stage = 0, slot = 0;
        uint32_t phase = 0, sphase = 0;
#define TASK_BEGIN
#define TASK_END
        T4_FOR_EACH_SEGMENT({
            int ok = 1;
            if (lane == 0) ok = mbar_wait(&sc_empty[slot], sphase ^ 1, abortp, wait_ns) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            uint32_t* sl = sc_ring + (size_t)slot * kSlotWords;
            // weight codes [tile][128 rows] (4 codes = one word per tile), rows past the matrix repeat the last row
            const int last_row = jb.n_rows - 1 - rb * 128;
            for (int i = lane; i < s.nt * 128; i += 32) {
                const int t = i >> 7, r = min(i & 127, last_row);
                cp4(&sl[t * 128 + (i & 127)], s.wsc + (size_t)r * jb.wscale_ld + t * 4);
            }
            for (int i = lane; i < s.nt * 16; i += 32) {
                const int t = i >> 4, c = i & 15;
                if (c < rows) cp4(&sl[kMaxSegTiles * 128 + t * 16 + c], s.asc + (size_t)c * jb.ascale_ld + t * 4);
            }
            if (s.coef && lane < rows) cp4(&sl[kMaxSegTiles * 144 + lane], s.coef + lane);
            cp_arrive(&sc_full[slot]);
            if (++slot == kScSlots) { slot = 0; sphase ^= 1; }
            if (lane == 0) {
                const CUtensorMap* wmap = reinterpret_cast<const CUtensorMap*>(&jb.tmap4);
                const CUtensorMap* amap = reinterpret_cast<const CUtensorMap*>(&jb.act_tmap);
                for (int t = 0; t < s.nt; t += kUnit) {
                    const int n2 = min(kUnit, s.nt - t);
                    if (!mbar_wait(&acc_full[stage], phase ^ 1, abortp, wait_ns)) break;  // the MMAs of the stage's last unit are done
                    uint8_t* st = ring + (size_t)stage * kStageBytes;
                    mbar_expect_tx(&full[stage], n2 * kTxBytes);
                    for (int i = 0; i < n2; ++i) {
                        tma_load_3d(st + i * kABytes, wmap, (s.t0 + t + i) * 128, s.row0, s.c2, &full[stage]);                    // elements
                        tma_load_3d(st + kUnit * kABytes + i * kBBytes, amap, (s.t0 + t + i) * 128, 0, s.aset, &full[stage]);  // bytes
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
            __syncwarp();
        })
#undef TASK_BEGIN
#undef TASK_END
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
#define TASK_BEGIN
#define TASK_END
            T4_FOR_EACH_SEGMENT({
                for (int t = 0; t < s.nt; t += kUnit) {
                    const int n2 = min(kUnit, s.nt - t);
                    if (!mbar_wait(&full[stage], phase, abortp, wait_ns)) break;
                    if (!mbar_wait(&acc_empty[stage], phase ^ 1, abortp, wait_ns)) break;
                    fence_after();
                    const uint32_t sa = smem_u32(ring + (size_t)stage * kStageBytes);
                    for (int i = 0; i < n2; ++i) {
                        const uint64_t adesc = desc_sw128(sa + i * kABytes), bdesc = desc_sw128(sa + kUnit * kABytes + i * kBBytes);
#pragma unroll
                        for (int g = 0; g < 4; ++g)  // one 32-value scale group per MMA, 32 bytes further along K
                            mma_f8f6f4(tmem_base + stage * (64 * kUnit) + i * 64 + g * 16, adesc + 2 * g, bdesc + 2 * g, kIdesc);
                    }
                    commit(&acc_full[stage]);
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            })
#undef TASK_BEGIN
#undef TASK_END
        }
    } else {
        // ------------------------------------------------------------ epilogue (TMEM lanes 32 * (warp % 4) ..)
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        const uint32_t tmem_lane = tmem_base + ((uint32_t)(q * 32) << 16);
        int stage = 0, slot = 0;
        uint32_t phase = 0, sphase = 0;
        float total_acc[kMaxRows];
#define TASK_BEGIN \
        _Pragma("unroll") for (int c = 0; c < kMaxRows; ++c) total_acc[c] = 0.f;
#define TASK_END                                                                                              \
        if (!*abortp) {                                                                                       \
            const int out_row = rb * 128 + row_in_tile;                                                       \
            float* out = jb.out + (size_t)((jb.mode == MONO_JOB_EXPERT_UP ? u_up * jb.nsplit : 0) + ks) * jb.out_split_stride; \
            if (out_row < jb.n_rows) {                                                                        \
                _Pragma("unroll") for (int c = 0; c < kMaxRows; ++c)                                          \
                    if (c < rows) out[(size_t)c * jb.out_ld + out_row] = total_acc[c];                        \
            }                                                                                                 \
        }
        T4_FOR_EACH_SEGMENT({
            if (!mbar_wait(&sc_full[slot], sphase, abortp, wait_ns)) break;
            const uint32_t* sl = sc_ring + (size_t)slot * kSlotWords;
            // the segment's activation scales as floats, one private copy per warp (no cross-warp barrier):
            // asf[tile][row][group] = 2^(code - 127)
            float* asf = asf_all + (size_t)q * kMaxSegTiles * 64;
            __syncwarp();
            for (int i = lane; i < s.nt * 16; i += 32) {
                const uint32_t a4 = sl[kMaxSegTiles * 128 + i];
                float4 f;
                f.x = __uint_as_float((a4 & 0xFFu) << 23);
                f.y = __uint_as_float(((a4 >> 8) & 0xFFu) << 23);
                f.z = __uint_as_float(((a4 >> 16) & 0xFFu) << 23);
                f.w = __uint_as_float((a4 >> 24) << 23);
                reinterpret_cast<float4*>(asf)[i] = f;
            }
            __syncwarp();
            float seg_acc[kMaxRows];
#pragma unroll
            for (int c = 0; c < kMaxRows; ++c) seg_acc[c] = 0.f;
            for (int t = 0; t < s.nt; t += kUnit) {
                const int n2 = min(kUnit, s.nt - t);
                if (!mbar_wait(&acc_full[stage], phase, abortp, wait_ns)) break;
                fence_after();
#pragma unroll
                for (int i = 0; i < kUnit; ++i) {
                    if (i < n2) {
                        uint32_t d[64];
                        ld64(tmem_lane + stage * (64 * kUnit) + i * 64, d);
                        if (i == n2 - 1) {  // the unit's accumulators are in registers: the MMA thread may reuse them
                            fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&acc_empty[stage]);
                        }
                        // this row's weight scales of the tile: 2^(code - 127); the product with an activation scale is exact
                        const uint32_t w4 = sl[(t + i) * 128 + row_in_tile];
                        const float u0 = __uint_as_float((w4 & 0xFFu) << 23), u1 = __uint_as_float(((w4 >> 8) & 0xFFu) << 23);
                        const float u2 = __uint_as_float(((w4 >> 16) & 0xFFu) << 23), u3 = __uint_as_float((w4 >> 24) << 23);
#pragma unroll
                        for (int c = 0; c < kMaxRows; ++c) {
                            if (c < rows) {
                                const float4 a = reinterpret_cast<const float4*>(asf)[(t + i) * 16 + c];
                                float v = __uint_as_float(d[c]) * (u0 * a.x);
                                v += __uint_as_float(d[16 + c]) * (u1 * a.y);
                                v += __uint_as_float(d[32 + c]) * (u2 * a.z);
                                v += __uint_as_float(d[48 + c]) * (u3 * a.w);
                                seg_acc[c] += v;
                            }
                        }
                    }
                }
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
#pragma unroll
            for (int c = 0; c < kMaxRows; ++c)
                if (c < rows) total_acc[c] += seg_acc[c] * (s.coef ? __uint_as_float(sl[kMaxSegTiles * 144 + c]) : 1.f);
            __syncwarp();
            if (lane == 0) mbar_arrive(&sc_empty[slot]);
            if (++slot == kScSlots) { slot = 0; sphase ^= 1; }
        })
#undef TASK_BEGIN
#undef TASK_END
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    }
#undef T4_FOR_EACH_SEGMENT
    fence_before();
    __syncthreads();
    if (abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before the CTA's memory goes
        if (tid == 0 && !guard_failed(p.a.guard)) guard_fail(p.a.guard, MONO_ERR_DEADLINE, 102);
    }
    if (warp == 1) {
        fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace tc4
}  // namespace mono

// Launches the tcgen05 MXFP4 kernel for an argument block that mono_gemv_launch has validated.
// Returns -100 when the block cannot take this path (the caller then uses the warp-MMA consumer).
int mono_gemv_tc4_launch(const mono_gemv_args* a, long tasks, cudaStream_t st) {
    using namespace mono;
    for (int j = 0; j < a->njobs; ++j) {
        const mono_gemv_job& jb = a->job[j];
        const unsigned long long* w4 = reinterpret_cast<const unsigned long long*>(&jb.tmap4);
        const unsigned long long* wa = reinterpret_cast<const unsigned long long*>(&jb.act_tmap);
        unsigned long long any4 = 0, anya = 0;
        for (int i = 0; i < 16; ++i) { any4 |= w4[i]; anya |= wa[i]; }
        const int seg = jb.mode == MONO_JOB_EXPERT_DOWN ? jb.k_tiles : (jb.split_tiles < jb.k_tiles ? jb.split_tiles : jb.k_tiles);
        if (!any4 || !anya || !jb.act_natural || jb.planes != 1 || jb.rb_per_mat != 0 || 2 * seg > tc4::kMaxSegTiles ||
            (jb.wscale_ld & 3) || (jb.ascale_ld & 3))
            return -100;
    }
    tc4::Params p;
    p.a = *a;
    const size_t smem = 1024 + (size_t)tc4::kStages * tc4::kStageBytes + (size_t)tc4::kScSlots * tc4::kSlotWords * 4 +
                        4 * tc4::kMaxSegTiles * 64 * sizeof(float) + 512;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        cudaError_t e = cudaFuncSetAttribute(tc4::gemv_tc4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        mono::attr_done(attr_once);
    }
    int grid = a->max_ctas > 0 ? a->max_ctas : mono_sm_count();
    if (grid > tasks) grid = (int)tasks;
    if (grid < 1) grid = 1;
    cudaError_t e = launch_k(tc4::gemv_tc4_kernel, grid, tc4::kThreads, smem, st, p);
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}
