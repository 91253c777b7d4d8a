// 4-bit weight-streaming GEMV on the block-scaled tensor-core kinds, one kernel body for two formats:
//
//   NVFP4  E2M1 weights x E2M1 activations, one unsigned E4M3 scale per 16 values on both operands, through
//          tcgen05.mma.kind::mxf4nvf4.block_scale (16-value blocks, K = 64 per MMA); the weights' f32 tensor scale is
//          applied to a task's f32 sum in the epilogue.  The format of MiniMax-M3.1-Flash's experts, which the
//          reference leaves to SGLang's MoE runner (minimax_m31/spec.py:117-121).
//   MXFP4  E2M1 weights x E4M3 activations, one E8M0 code per 32 values on both operands, through
//          tcgen05.mma.kind::mxf8f6f4.block_scale (K = 32 per MMA): the reference's W4A8 expert arithmetic
//          (minimax_m3/gfx950/post_attn.py:1304-1314, glm53_flash/gfx950/kernel.py:4025-4392; E8M0 rule
//          common/mx.py:27-39).  Same sums as gemv_tc4bs.cu, which this kernel replaces where the weight's scale
//          codes have been repacked (mono_gemv_job.wscale_t).
//
// Task list, outputs and job modes are those of the other GEMV kernels.
//
// Operands.  A unit is one TMA box of weights: 128 rows x 16 KB of shared memory.  NVFP4: both operands of the MMA
// are packed 4-bit values, 64 per MMA, so a 128-byte-wide box of packed bytes (256 k values) is the operand as TMA
// delivers it (128-byte swizzle) and the ring holds nothing but HBM bytes.  MXFP4 next to 8-bit activations: the MMA
// reads 4-bit values padded to 16 per 16 bytes, and TMA writes that form itself from a tensor map of 4-bit elements
// (128 k values per box, 8 KB fetched for 16 KB written): no warp touches the nibbles, but a ring slot holds half as
// many HBM bytes.  The ring's slots (8 or 10) are free again when the MMAs that read them are done.
//
// Scale factors.  An MMA reads 4 scale bytes per row from 4 TMEM columns per operand: row r's bytes are column r / 32
// of lane r % 32 (NVFP4: the four 16-value blocks of the MMA; MXFP4: the four 32-value groups of the unit, one per
// MMA, picked by the instruction descriptor).  tcgen05.cp (32 lanes x 128 bits, repeated for the four lane quarters)
// brings them from a 512-byte block of shared memory laid out as bytes [(r % 32) * 16 + (r / 32) * 4 + block].  The
// weights' scale bytes are stored in that order (mono_gemv_job.wscale_t, a one-time repack when the weight is
// bound): those of a (row block, unit) arrive by one bulk copy beside the unit's weights.  (Gathered from row-major
// rows by warps of the kernel, a segment's bytes took 2.2 - 2.8 us under load, as long as its MMAs.)  The
// activations' bytes (16 rows: the first 16 lanes of column 0, so their blocks overlap, 256 bytes apart) are gathered
// by four scale warps, segment by segment in turn, each into a slot of its own, up to four segments ahead of the MMA
// threads.  Every scale byte the MMA can see is a valid number from the start (1.0).
//
// Issue rate.  Per unit: four MMAs and two (MXFP4) or eight (NVFP4) scale copies, about 70 cycles each for the
// issuing thread.  Two threads of two warps issue in turn, unit by unit, each into an accumulator of its own; the
// epilogue adds the two.  The issuing threads do not walk the task list (a single thread needs about 1 us for the
// divisions and address arithmetic of a segment): the scale warps leave each segment's unit count in its slot.
//
// 384 threads: one thread each of warps 0 and 11 issues the TMA copies, one thread each of warps 1 and 7 issues
// tcgen05.cp + MMA, warps 2..5 own the 128 TMEM lanes (epilogue), warps 6, 8, 9, 10 stage the activations' scale bytes.  Every wait is bounded; TMEM is freed on every
// exit path.
#include "mono_common.cuh"

extern void mono_set_error(const char* fmt, ...);

namespace mono {
namespace nvf4 {

constexpr int kThreads = 384;
constexpr int kPackBytes = 128 * 128;   // a unit of weights in shared memory: 128 rows x 128 bytes
constexpr int kBBytes = 16 * 128;       // the unit's activations: 16 rows x 128 bytes
constexpr int kMmas = 4;                // MMAs per unit
constexpr int kSfBlock = 512;           // scale bytes in the order tcgen05.cp wants: 128 rows x 4
constexpr int kScWarps = 4;             // scale warps: warp i takes segments i, i + 4, ...
constexpr int kScSlots = kScWarps;      // ... into a slot of its own (one writer per slot: its uses follow one another)
constexpr int kSfbStep = 256;           // activations: blocks half a block apart
constexpr int kAccCols = 16;            // one accumulator: 16 columns (the step's rows); [2 segments in turn][2 issuers]
constexpr int kSfCol = 4 * kAccCols;    // per issuer 64 columns: [2 units in turn][4 MMAs][weights 4 | activations 4 ... ]
constexpr int kTmemCols = 256;

// What differs between the two formats
template <bool NV>
struct Fmt {
    static constexpr int kUnitK = NV ? 256 : 128;             // k values per unit
    static constexpr int kSfaUnit = NV ? kMmas * kSfBlock : kSfBlock;  // weight scale bytes per (row block, unit)
    static constexpr int kSfbPerUnit = NV ? kMmas : 1;        // activation scale blocks per unit
    static constexpr int kAscBytes = NV ? 16 : 4;             // activation scale bytes per row and unit
    static constexpr int kTxBytes = (NV ? kPackBytes : kPackBytes / 2) + kBBytes + kSfaUnit;  // bytes TMA fetches per unit
    static constexpr int kStageBytes = (kPackBytes + kBBytes + kSfaUnit + 1023) & ~1023;
    // Two rings of kStages / 2 slots: ring i is filled by producing thread i and read by issuing thread i only, so a
    // slot's uses follow one another in one thread on either side.  (A waiter only knows a barrier's parity: were a
    // slot's previous use pending in ANOTHER thread's queue, a barrier two uses behind would look like one that is
    // ready.)
    static constexpr int kStages = NV ? 8 : 10;
    static constexpr int kRing = kStages / 2;
    static_assert(kStages % 2 == 0, "one ring per issuing thread");
    static constexpr int kMaxSegUnits = NV ? 8 : 16;          // 2048 k values per segment
    static constexpr int kSfbBytes = kMaxSegUnits * kSfbPerUnit * kSfbStep + kSfBlock / 2;
    static constexpr int kSlotBytes = kSfbBytes + 128;        // + 16 route coefficients, the tensor scale and the unit count
    static constexpr int kAloneUnits = NV ? 2 : 4;            // a segment of so few units has one issuing thread
    static constexpr uint32_t kOne4 = NV ? 0x38383838u : 0x7F7F7F7Fu;  // four scale bytes of 1.0 (E4M3 / E8M0)
    static constexpr size_t kSmem = 1024 + (size_t)kStages * kStageBytes + (size_t)kScSlots * kSlotBytes + 512;
};

struct Params {
    mono_gemv_args a;
};

MONO_TL_DECLARE(tl_nv)
#ifdef MONO_TIMELINE
// stamps of CTA 0's roles, units 32.. of the launch (steady state): row 140 + k, one column per unit
#define NV_TL(k, n) do { if (blockIdx.x == 0 && (n) >= 32 && (n) < 32 + MONO_TL_POINTS) tl_nv[140 + (k)][(n) - 32] = globaltimer_ns(); } while (0)
#else
#define NV_TL(k, n) do { } while (0)
#endif

struct Seg {
    int c2, row0, t0, nt, aset;  // t0, nt in units
    const uint8_t* asc;
    const uint8_t* wsc;
    const float* coef;
    const float* gp;  // the matrix's tensor scale (or null)
};

__device__ __forceinline__ int nrb_of(const mono_gemv_job& j) { return (j.n_rows + 127) >> 7; }

// What a task's segments share: computed once per task, so that a segment of a down projection (an expert of a few
// hundred values) costs a role a table lookup and a handful of multiply-adds.
struct TaskC {
    int mode, row0, t0, nt;
    const uint8_t* asc0;  // + aset * ascale_seg_stride
    const uint8_t* wsc0;  // + mat * wscale_mat_stride
    long a_stride, w_stride;
    const float* coef;
    const float* wglobal;
    const int32_t* expert_list;
};

// units of the job's K: NVFP4 counts k_tiles in units; MXFP4 in 128-byte tiles of nibbles = two units
template <bool NV>
__device__ __forceinline__ int units_of(const mono_gemv_job& j) { return NV ? j.k_tiles : (j.k_tiles4 > 0 ? j.k_tiles4 : 2 * j.k_tiles); }

template <bool NV>
__device__ __forceinline__ TaskC make_task(const mono_gemv_job& j, int rb, int ks) {
    TaskC t;
    t.mode = j.mode;
    t.row0 = j.row_off + rb * 128;
    const int total = units_of<NV>(j), per_split = (NV ? 1 : 2) * j.split_tiles;
    if (j.mode == MONO_JOB_EXPERT_DOWN) {
        t.t0 = 0;
        t.nt = total;
    } else {
        t.t0 = ks * per_split;
        t.nt = min(per_split, total - t.t0);
    }
    t.asc0 = j.ascale_e8 + (size_t)t.t0 * Fmt<NV>::kAscBytes;
    t.wsc0 = j.wscale_t + (size_t)(t.row0 >> 7) * j.wscale_t_ld + (size_t)t.t0 * Fmt<NV>::kSfaUnit;
    t.a_stride = j.ascale_seg_stride;
    t.w_stride = j.wscale_t_mat_stride;
    t.coef = j.coef;
    t.wglobal = j.wglobal;
    t.expert_list = j.expert_list;
    return t;
}

__device__ __forceinline__ Seg make_seg(const TaskC& t, int u, const int* elist) {
    Seg s;
    const int mat = t.mode == MONO_JOB_DENSE ? 0 : ((u < 128) ? elist[u] : t.expert_list[u]);
    const bool down = t.mode == MONO_JOB_EXPERT_DOWN;
    s.c2 = mat;
    s.row0 = t.row0;
    s.t0 = t.t0;
    s.nt = t.nt;
    s.aset = down ? u : 0;
    s.coef = (down && t.coef) ? t.coef + (size_t)u * kMaxRows : nullptr;
    s.asc = t.asc0 + (size_t)s.aset * t.a_stride;
    s.wsc = t.wsc0 + (size_t)mat * t.w_stride;
    s.gp = t.wglobal ? t.wglobal + mat : nullptr;
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
// 32 lanes x 128 bits of shared memory to 4 TMEM columns, the same 32 rows in each of the four lane quarters
__device__ __forceinline__ void cp_sf(uint32_t tmem_col, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void mma_nvf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
__device__ __forceinline__ void mma_mxf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
// 32 TMEM columns (both issuers' accumulators of a segment) of this thread's lane
__device__ __forceinline__ void ld32(uint32_t taddr, uint32_t r[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// K-major tile with 128-byte rows and the 128-byte swizzle: groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// A scale block: 32 rows of 16 bytes, no swizzle; groups of 8 rows 128 bytes apart (one 16-byte piece along K)
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(16 >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) | (1ull << 46);
}
// Block-scaled descriptor: A and B E2M1 (format 1 of this kind), both K-major, N = 16, unsigned E4M3 scales
// (scale-format bit 23 clear), M = 128; all four scale bytes of a column are used (scale ids 0)
constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | (0u << 23) | ((128u >> 4) << 24);
// MXFP4 x MXFP8: A E2M1 (format 5 of this kind), B E4M3 (format 0), E8M0 scales, N = 16, M = 128; group g of the
// unit: byte g of the scale columns for both operands
__device__ __forceinline__ uint32_t idesc_group(uint32_t g) {
    return (g << 4) | (5u << 7) | (0u << 10) | ((16u >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | (g << 29);
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <bool NV>
__device__ __forceinline__ void gemv_fp4_body(const Params& p) {
    using F = Fmt<NV>;
    constexpr int kStages = F::kStages, kStageBytes = F::kStageBytes, kSlotBytes = F::kSlotBytes, kSfbBytes = F::kSfbBytes;
    constexpr int kSfaUnit = F::kSfaUnit, kMaxSegUnits = F::kMaxSegUnits, kSfbPerUnit = F::kSfbPerUnit;
    constexpr uint32_t kOne4 = F::kOne4;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;                                    // kStages slots: weights, then activations
    uint8_t* sc_ring = ring + (size_t)kStages * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sc_ring + (size_t)kScSlots * kSlotBytes);
    uint64_t* full = bars;                      // TMA -> MMA: a slot's boxes have landed
    uint64_t* stage_free = full + kStages;      // MMA -> TMA: the MMAs that read the slot are done
    uint64_t* sc_full = stage_free + kStages;   // scale warp -> MMA / epilogue: a segment's scale bytes are staged
    uint64_t* sc_empty = sc_full + kScSlots;    // 2 issuers (unit count read) + 4 epilogue warps (coefficients read; the
                                                // accumulators they waited for were complete, so the issuers' copies from
                                                // the slot are done too)
    uint64_t* acc_full = sc_empty + kScSlots;   // [buffer][issuer] -> epilogue: that issuer's accumulator of the segment is complete
    uint64_t* acc_empty = acc_full + 4;         // 4 epilogue warps -> MMA
    __shared__ int abort_flag;
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_elist[MONO_GEMV_MAX_JOBS][128];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rows = p.a.rows;
    if (blockIdx.x < 140) MONO_TL(tl_nv, 0);
    if (tid == 0) {
        abort_flag = guard_failed(p.a.guard) ? 1 : 0;
        for (int i = 0; i < kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&stage_free[i], 1); }
        for (int i = 0; i < kScSlots; ++i) { mbar_init(&sc_full[i], 32); mbar_init(&sc_empty[i], 6); }
        for (int i = 0; i < 4; ++i) mbar_init(&acc_full[i], 1);
        for (int i = 0; i < 2; ++i) mbar_init(&acc_empty[i], 4);
        mbar_fence_init();
    }
    for (int i = tid; i < kScSlots * kSlotBytes / 4; i += kThreads) reinterpret_cast<uint32_t*>(sc_ring)[i] = kOne4;
    fence_proxy_async_smem();
    if (warp == 1) tmem_alloc(&tmem_base_s, kTmemCols);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_launch_dependents();
    if (blockIdx.x < 140) MONO_TL(tl_nv, 1);
    pdl_wait();
    if (blockIdx.x < 140) MONO_TL(tl_nv, 2);

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

// every role walks the same (task, segment) sequence
#define NV_FOR_EACH_SEGMENT(...)                                                                                \
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
        const TaskC tc = make_task<NV>(jb, rb, ks);                                                             \
        const int u_step = jb.nsplit;                                                                           \
        TASK_BEGIN                                                                                              \
        for (int sgi = 0; sgi < nseg && !*abortp; ++sgi) {                                                      \
            if (tc.mode == MONO_JOB_EXPERT_DOWN) u = ks + sgi * u_step;                                         \
            const Seg s = make_seg(tc, u, s_elist[j]);                                                          \
            __VA_ARGS__                                                                                         \
        }                                                                                                       \
        TASK_END                                                                                                \
    }

    if (warp == 0 || warp == 11) {
        // ------------------------------------------------------------ producers: weight boxes, activation tiles and weight
        // scales by TMA.  One thread needs about 0.3 us for a unit's wait and four instructions, which bounded the
        // MXFP4 launch (8 KB of HBM bytes per unit) at 3.1 TB/s.  Thread i feeds issuing thread i through ring i: the
        // units of its parity (launch-wide numbers) of a long segment, every unit of a short segment that is its
        // issuer's (see the issuers).
        if (lane == 0) {
            const int pid = warp == 0 ? 0 : 1;
            int n = 0, seg_no = 0, mine = 0;  // launch-wide unit and segment numbers; units this thread has copied
#define TASK_BEGIN
#define TASK_END
            NV_FOR_EACH_SEGMENT({
                // NVFP4: the weight as bytes, 128 per box row = 256 values; MXFP4: as 4-bit elements, 128 per box row,
                // which TMA pads to 128 bytes.  The box's first coordinate is unit * 128 in both (bytes / elements).
                const CUtensorMap* wmap = reinterpret_cast<const CUtensorMap*>(NV ? &jb.tmap : &jb.tmap4);
                const CUtensorMap* amap = reinterpret_cast<const CUtensorMap*>(&jb.act_tmap);
                // (L2 prefetch requests for a segment's later boxes, issued here before its first copy, made both
                // formats slower: 77.6 -> 87.3 us and 51.4 -> 56.7 us for the config-4 up/gate launch; the copies
                // themselves start later by the time this thread spends on the requests.)
                const bool alone = s.nt <= F::kAloneUnits;
                const bool skip = alone && (seg_no & 1) != pid;
                ++seg_no;
                for (int t = alone ? 0 : ((n + pid) & 1); t < s.nt && !skip; t += alone ? 1 : 2) {
                    const int un = n + t, stage = pid * F::kRing + mine % F::kRing;
                    const uint32_t phase = (uint32_t)(mine / F::kRing) & 1u;
                    ++mine;
                    (void)un;
                    NV_TL(0, un);
                    if (!mbar_wait(&stage_free[stage], phase ^ 1, abortp, wait_ns)) break;
                    NV_TL(1, un);
                    uint8_t* st = ring + (size_t)stage * kStageBytes;
                    // (a box that reaches past K reads zeros there and still counts its full size)
                    mbar_expect_tx(&full[stage], F::kTxBytes);
                    tma_load_3d(st, wmap, (s.t0 + t) * 128, s.row0, s.c2, &full[stage]);
                    tma_load_3d(st + kPackBytes, amap, (s.t0 + t) * 128, 0, s.aset, &full[stage]);
                    bulk_load(st + kPackBytes + kBBytes, s.wsc + (size_t)t * kSfaUnit, kSfaUnit, &full[stage]);
                    NV_TL(2, un);
                }
                n += s.nt;
            })
#undef TASK_BEGIN
#undef TASK_END
        }
    } else if (warp == 1 || warp == 7) {
        // ------------------------------------------------------------ scale copies + MMA: issuer `me` takes the launch's
        // units n = me, me + 2, ... and adds them into its own accumulator of the segment
        // The issuing threads do not walk the task list (a single thread needs about 1 us for the divisions and
        // address arithmetic of a segment, time in which no MMA is issued): the scale warps leave each segment's
        // unit count in its slot, and a count of zero ends the launch.
        // A segment of one or two units (a down projection of a narrow expert) belongs to ONE issuer, the segments
        // alternating between the two: the handshakes of a segment cost an issuing thread about as much as the twelve
        // instructions of a unit, so two threads sharing such a segment spent 1.3 us on it, while each taking every
        // other segment as a whole they overlap their handshakes.
        if (lane == 0) {
            const int me = warp == 1 ? 0 : 1;
            int slot = 0, n0 = 0, seg_no = 0;
            uint32_t sphase = 0, mine = 0;
            for (;;) {
                if (!mbar_wait(&sc_full[slot], sphase, abortp, wait_ns)) break;
                const int word = reinterpret_cast<const volatile int*>(sc_ring + (size_t)slot * kSlotBytes + kSfbBytes)[kMaxRows + 1];
                const int nt = word & 0xFF, nm_last = word >> 8;  // units; MMAs of the last unit
                if (nt <= 0) break;
                mbar_arrive(&sc_empty[slot]);  // this thread has read the slot's words (its copies: see sc_empty)
                const int buf = seg_no & 1;
                const uint32_t aphase = (uint32_t)(seg_no >> 1) & 1u;
                const bool alone = nt <= F::kAloneUnits;  // the segment has one owner: issuer `buf`
                if (me == 0) NV_TL(13, n0);
                // (every issuer waits for every buffer turn, owner or not: the parities of a barrier it skipped
                // for two turns would no longer tell it anything)
                if (!mbar_wait(&acc_empty[buf], aphase ^ 1, abortp, wait_ns)) break;
                if (me == 0) NV_TL(7, n0);
                if (me == 0 && n0 == 0 && blockIdx.x < 140) MONO_TL_AT(tl_nv, 5);
                bool ok = true;
                if (!alone || buf == me) {
                    fence_after();
                    const uint32_t sl = smem_u32(sc_ring + (size_t)slot * kSlotBytes);
                    const uint32_t acc = tmem_base + (buf * 2 + me) * kAccCols;
                    uint32_t accumulate = 0;
                    // shared segment: the units of this issuer's parity (launch-wide numbers); own segment: all
                    for (int t = alone ? 0 : ((n0 + me) & 1); t < nt; t += alone ? 1 : 2) {
                        const int n = n0 + t, st_now = me * F::kRing + (int)(mine % F::kRing);  // ring `me`, its units in order
                        const uint32_t ph_now = (mine / F::kRing) & 1u;
                        (void)n;
                        NV_TL(3, n);
                        if (!mbar_wait(&full[st_now], ph_now, abortp, wait_ns)) { ok = false; break; }
                        NV_TL(4, n);
                        fence_after();
                        const uint32_t sa = smem_u32(ring + (size_t)st_now * kStageBytes);
                        const uint64_t adesc = desc_sw128(sa), bdesc = desc_sw128(sa + kPackBytes);
                        // (the tensor pipe runs a thread's copies and MMAs in the order it issued them; the column sets
                        // alternate from unit to unit all the same)
                        const uint32_t set = tmem_base + kSfCol + me * 64 + (mine & 1) * 32;
                        ++mine;
                        const int nm = t == nt - 1 ? nm_last : kMmas;  // K may end inside the segment's last unit
                        if (NV) {
#pragma unroll
                            for (int m = 0; m < kMmas; ++m) {  // 64 values per MMA, 32 bytes further along K
                                if (m >= nm) break;
                                const int blk = t * kMmas + m;
                                const uint32_t sfa = set + m * 8, sfb = sfa + 4;
                                cp_sf(sfa, desc_sf(sa + kPackBytes + kBBytes + m * kSfBlock));
                                cp_sf(sfb, desc_sf(sl + blk * kSfbStep));
                                mma_nvf4(acc, adesc + 2 * m, bdesc + 2 * m, kIdesc, sfa, sfb, accumulate);
                                accumulate = 1;
                            }
                        } else {
                            const uint32_t sfa = set, sfb = set + 4;
                            cp_sf(sfa, desc_sf(sa + kPackBytes + kBBytes));
                            cp_sf(sfb, desc_sf(sl + t * kSfbStep));
#pragma unroll
                            for (uint32_t g = 0; g < (uint32_t)kMmas; ++g) {  // one 32-value group per MMA, 32 bytes further along K
                                mma_mxf4(acc, adesc + 2 * g, bdesc + 2 * g, idesc_group(g), sfa, sfb, accumulate);
                                accumulate = 1;
                            }
                        }
                        commit(&stage_free[st_now]);
                        NV_TL(5, n);
                    }
                    if (!ok) break;
                    NV_TL(6, n0 + nt - 1);
                    commit(&acc_full[buf * 2 + me]);
                    if (me == 0) NV_TL(18, n0 + nt - 1);
                }
                n0 += nt;
                ++seg_no;
                if (++slot == kScSlots) { slot = 0; sphase ^= 1; }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue (TMEM lanes 32 * (warp % 4) ..)
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        const uint32_t tmem_lane = tmem_base + ((uint32_t)(q * 32) << 16);
        int slot = 0, n = 0, seg_no = 0;
        uint32_t sphase = 0, fphase = 0;  // fphase: bit (buffer * 2 + issuer) = parity of that accumulator's next turn
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
        NV_FOR_EACH_SEGMENT({
            if (!mbar_wait(&sc_full[slot], sphase, abortp, wait_ns)) break;
            if (tid == 64) NV_TL(11, n);
            // whose accumulators hold this segment: its owner's (one or two units), else both issuers'
            const int buf = seg_no & 1;
            const bool alone = s.nt <= F::kAloneUnits, w0 = !alone || buf == 0, w1 = !alone || buf == 1;
            ++seg_no;
            bool got = true;
            if (w0) { got = mbar_wait(&acc_full[buf * 2], (fphase >> (buf * 2)) & 1u, abortp, wait_ns); fphase ^= 1u << (buf * 2); }
            if (got && w1) { got = mbar_wait(&acc_full[buf * 2 + 1], (fphase >> (buf * 2 + 1)) & 1u, abortp, wait_ns); fphase ^= 1u << (buf * 2 + 1); }
            if (!got) break;
            if (tid == 64) NV_TL(12, n);
            fence_after();
            uint32_t d[32];
            ld32(tmem_lane + buf * 2 * kAccCols, d);
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            n += s.nt;
            if (tid == 64) NV_TL(15, n - s.nt);
            const float* coef = reinterpret_cast<const float*>(sc_ring + (size_t)slot * kSlotBytes + kSfbBytes);
            const float g = coef[kMaxRows];
#pragma unroll
            for (int c = 0; c < kMaxRows; ++c)
                if (c < rows)
                    total_acc[c] += ((w0 ? __uint_as_float(d[c]) : 0.f) + (w1 ? __uint_as_float(d[kAccCols + c]) : 0.f)) * g * coef[c];
            __syncwarp();
            if (lane == 0) mbar_arrive(&sc_empty[slot]);
            if (++slot == kScSlots) { slot = 0; sphase ^= 1; }
        })
#undef TASK_BEGIN
#undef TASK_END
    } else if (warp == 6 || (warp >= 8 && warp <= 10)) {
        // ------------------------------------------------------------ scale warps: a segment's activation scale bytes,
        // route coefficients, tensor scale and unit count, up to four segments ahead.  A segment costs its warp a
        // memory round trip (1 - 2 us under load), more than the MMAs of a short segment (a down projection of 384
        // values: two units, 0.8 us): four warps take the segments in turn, so four round trips overlap.
        const int sw = warp == 6 ? 0 : warp - 7;
        int seg_no = 0, tl_n = 0;
        (void)tl_n;
#define TASK_BEGIN
#define TASK_END
        NV_FOR_EACH_SEGMENT({
            const int slot = seg_no % kScSlots;
            const uint32_t sphase = (uint32_t)(seg_no / kScSlots) & 1u;
            const bool mine = (seg_no % kScWarps) == sw;
            ++seg_no;
            if (!mine) { tl_n += s.nt; continue; }
            int ok = 1;
            if (lane == 0 && sw == 0) NV_TL(8, tl_n);
            if (lane == 0) ok = mbar_wait(&sc_empty[slot], sphase ^ 1, abortp, wait_ns) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane == 0 && sw == 0) NV_TL(9, tl_n);
            uint8_t* sl = sc_ring + (size_t)slot * kSlotBytes;
            // row c's four bytes of MMA m are the first four bytes of row c of the MMA's block (rows past the step:
            // 1.0); lanes 0..15 take the even units, 16..31 the odd ones; every load is issued before the first store
            const int c = lane & 15;
            const uint8_t* arow = s.asc + (size_t)min(c, rows - 1) * jb.ascale_ld;
            uint32_t a4[kMaxSegUnits / 2][kSfbPerUnit];  // NVFP4: a row's 16 bytes of a unit; MXFP4: its 4
#pragma unroll
            for (int k = 0; k < kMaxSegUnits / 2; ++k) {
                const uint8_t* src = arow + min((lane >> 4) + 2 * k, s.nt - 1) * F::kAscBytes;
                if (NV) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
                    a4[k][0] = v.x; a4[k][kSfbPerUnit > 1 ? 1 : 0] = v.y; a4[k][kSfbPerUnit > 2 ? 2 : 0] = v.z; a4[k][kSfbPerUnit > 3 ? 3 : 0] = v.w;
                } else {
                    a4[k][0] = __ldg(reinterpret_cast<const uint32_t*>(src));
                }
            }
            float cf_v = 1.f;
            if (s.coef && lane < rows) cf_v = __ldg(s.coef + lane);
#pragma unroll
            for (int k = 0; k < kMaxSegUnits / 2; ++k) {
                const int t = (lane >> 4) + 2 * k;
                if (t < s.nt) {
                    uint8_t* blk = sl + (size_t)t * kSfbPerUnit * kSfbStep + c * 16;
                    const bool live = c < rows;
#pragma unroll
                    for (int m = 0; m < kSfbPerUnit; ++m) *reinterpret_cast<uint32_t*>(blk + m * kSfbStep) = live ? a4[k][m] : kOne4;
                }
            }
            {
                float* cf = reinterpret_cast<float*>(sl + kSfbBytes);
                if (lane < kMaxRows) cf[lane] = cf_v;
                if (lane == kMaxRows) cf[lane] = s.gp ? __ldg(s.gp) : 1.f;
                if (lane == kMaxRows + 1) {  // for the issuing threads: units, and the MMAs of the last unit (K may end inside it)
                    int nm_last = kMmas;
                    if (NV) {
                        const int k_mmas = jb.k_tiles4 > 0 ? jb.k_tiles4 : jb.k_tiles * kMmas;
                        nm_last = max(1, min(kMmas, k_mmas - (s.t0 + s.nt - 1) * kMmas));
                    }
                    reinterpret_cast<int*>(cf)[lane] = s.nt | (nm_last << 8);
                }
            }
            fence_proxy_async_smem();  // the copies to TMEM read these bytes through the async proxy
            mbar_arrive(&sc_full[slot]);
            if (lane == 0 && sw == 0) NV_TL(10, tl_n);
            tl_n += s.nt;
        })
#undef TASK_BEGIN
#undef TASK_END
        // the end marker: a slot with a unit count of zero, from the warp whose turn it is
        if (!*abortp && (seg_no % kScWarps) == sw) {
            const int slot = seg_no % kScSlots;
            const uint32_t sphase = (uint32_t)(seg_no / kScSlots) & 1u;
            int ok = 1;
            if (lane == 0) ok = mbar_wait(&sc_empty[slot], sphase ^ 1, abortp, wait_ns) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (ok) {
                if (lane == kMaxRows + 1) reinterpret_cast<int*>(sc_ring + (size_t)slot * kSlotBytes + kSfbBytes)[lane] = 0;
                mbar_arrive(&sc_full[slot]);
            }
        }
    }
#undef NV_FOR_EACH_SEGMENT
    if (blockIdx.x < 140) MONO_TL(tl_nv, 3);  // the producer has issued its last unit
    fence_before();
    __syncthreads();
    if (blockIdx.x < 140) MONO_TL(tl_nv, 4);
    if (abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before the CTA's memory goes
        if (tid == 0 && !guard_failed(p.a.guard)) guard_fail(p.a.guard, MONO_ERR_DEADLINE, 104);
    }
    if (warp == 1) {
        fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

__global__ void __launch_bounds__(kThreads, 1) gemv_nvf4_kernel(const __grid_constant__ Params p) { gemv_fp4_body<true>(p); }
__global__ void __launch_bounds__(kThreads, 1) gemv_mxf4_kernel(const __grid_constant__ Params p) { gemv_fp4_body<false>(p); }

}  // namespace nvf4
}  // namespace mono

#ifdef MONO_TIMELINE
extern "C" int mono_timeline_read_nvf4(unsigned long long* out, int* ctas, int* points) {
    *ctas = MONO_TL_CTAS;
    *points = MONO_TL_POINTS;
    return (int)cudaMemcpyFromSymbol(out, mono::nvf4::tl_nv, sizeof(unsigned long long) * MONO_TL_CTAS * MONO_TL_POINTS);
}
#endif

// Launches the kernel for an argument block that mono_gemv_launch has validated (wkind MONO_W_NVFP4 or MONO_W_MXFP4).
// Returns -100 when the block does not have what this kernel needs.
template <bool NV>
static int fp4_launch(const mono_gemv_args* a, long tasks, cudaStream_t st) {
    using namespace mono;
    using F = nvf4::Fmt<NV>;
    for (int j = 0; j < a->njobs; ++j) {
        const mono_gemv_job& jb = a->job[j];
        const unsigned long long* wa = reinterpret_cast<const unsigned long long*>(&jb.act_tmap);
        const unsigned long long* wb = reinterpret_cast<const unsigned long long*>(NV ? &jb.tmap : &jb.tmap4);
        unsigned long long anya = 0, anyb = 0;
        for (int i = 0; i < 16; ++i) { anya |= wa[i]; anyb |= wb[i]; }
        const int units = NV ? jb.k_tiles : (jb.k_tiles4 > 0 ? jb.k_tiles4 : 2 * jb.k_tiles);
        const int per_split = (NV ? 1 : 2) * jb.split_tiles;
        const int seg = jb.mode == MONO_JOB_EXPERT_DOWN ? units : (per_split < units ? per_split : units);
        if (!anya || !anyb || jb.planes != 1 || jb.rb_per_mat != 0 || seg > F::kMaxSegUnits || jb.feeds_job || (!NV && !jb.act_natural) ||
            !jb.wscale_t || (jb.row_off & 127) || (jb.wscale_t_ld & 15) || (jb.ascale_ld & 3) ||
            (reinterpret_cast<uintptr_t>(jb.wscale_t) & 15) || (reinterpret_cast<uintptr_t>(jb.ascale_e8) & 15) ||
            (jb.wscale_t_mat_stride & 15) || (jb.ascale_seg_stride & 15) || (NV && (jb.ascale_ld & 15)) ||
            (long)jb.wscale_t_ld < (long)units * F::kSfaUnit || (long)jb.ascale_ld < (long)units * F::kAscBytes ||
            jb.wscale_t_mat_stride < (long)((jb.row_off + jb.n_rows + 127) / 128) * jb.wscale_t_ld)
            return -100;
    }
    nvf4::Params p;
    p.a = *a;
    auto kernel = NV ? nvf4::gemv_nvf4_kernel : nvf4::gemv_mxf4_kernel;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d (one instance of this function per format)
    if (mono::attr_needed(attr_once)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F::kSmem);
        if (e != cudaSuccess) return (int)e;
        mono::attr_done(attr_once);
    }
    int grid = a->max_ctas > 0 ? a->max_ctas : mono_sm_count();
    if (grid > tasks) grid = (int)tasks;
    if (grid < 1) grid = 1;
    cudaError_t e = launch_k(kernel, grid, nvf4::kThreads, F::kSmem, st, p);
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

int mono_gemv_nvf4_launch(const mono_gemv_args* a, long tasks, cudaStream_t st) { return fp4_launch<true>(a, tasks, st); }
int mono_gemv_mxf4_launch(const mono_gemv_args* a, long tasks, cudaStream_t st) { return fp4_launch<false>(a, tasks, st); }
