// MXFP4 weight-streaming GEMV on the block-scaled tensor-core kind: E2M1 weights x E4M3 activations through
// tcgen05.mma.kind::mxf8f6f4.block_scale, both operands' E8M0 group-32 codes read by the MMA itself from
// tensor memory.  A task's whole K run accumulates in ONE TMEM accumulator (128 rows x 16 columns of f32); the
// epilogue reads it once per segment and only applies the routed expert's coefficient.
//
// Same contract and task list as gemv_tc4.cu (which issues kind::f8f6f4 once per 32-value group into separate
// accumulators and scales in the epilogue); reference arithmetic: the scaled-MFMA expert stages of
// minimax_m3/gfx950/post_attn.py:1304-1314 and glm53_flash/gfx950/kernel.py:4025-4392, E8M0 rule
// common/mx.py:27-39.  Difference in the last bits: the products of a group are scaled and added inside the
// tensor core, so a task's sum is not the f32 sum, group by group in k order, that gemv_tc4.cu and the CPU
// restatement form; the results agree to f32 rounding of a K-long sum (the tests state the tolerance).
//
// Scale factors.  The MMA reads the codes of a 128-element k tile (4 groups) from 4 TMEM columns per operand:
// row r's four codes are the four bytes of column r / 32 in lane r % 32; the instruction descriptor's a_sf_id /
// b_sf_id pick the byte (the group).  tcgen05.cp (32 lanes x 128 bits, repeated for the four lane quarters)
// brings codes from a 512-byte block of shared memory in exactly that order: bytes
// [(r % 32) * 16 + (r / 32) * 4 + group].  A scale warp gathers the codes from their row-major home in global
// memory into such blocks, one segment ahead of the MMA thread: one block per tile for the weights (128 rows).
// The activations have 16 rows (the first 16 lanes of column 0), so their blocks overlap: tile t's block starts
// 256 bytes after tile t - 1's, and its unused second half is the next tile's first.  (The MMA wants a scale
// address at a multiple of four columns: several tiles cannot share one copy's columns.)  The scale warp orders
// its generic-proxy stores against the async proxy before it signals them.
//
// Bytes in flight.  The MMA reads 4-bit operands from shared memory in a padded form (16 values in the low 8 bytes
// of every 16), twice the size of the packed nibbles.  A ring of tiles in that form holds too few HBM bytes to
// cover the DRAM latency at full bandwidth (8 tiles = 64 KB per SM streamed at 3.0 - 3.8 TB/s in a copy-only
// test).  So TMA brings the nibbles PACKED (plain bytes, 128 rows x 128 bytes = two k tiles per box, 128-byte
// swizzle) into a deep staging ring, and four converter warps spread each box into one of two padded operand
// buffers (8 bytes -> the low half of a 16-byte slot, the operand's 128-byte swizzle applied) just before the
// MMAs read it; a staging slot is free again as soon as it has been spread, not when its MMAs are done.
//
// Issue rate.  An MMA of this kind covers 32 k values: four MMAs and two scale copies per 8 KB of weights, and a
// thread issues one such instruction in about 90 cycles (measured: 0.58 us for the twelve of a two-tile unit).  Two
// threads of two warps therefore issue in turn, unit by unit, each into an accumulator of its own; the epilogue
// adds the two.
//
// 384 threads: warp 0 TMA, one thread each of warps 1 and 11 issues tcgen05.cp + MMA, warps 2..5 own the 128 TMEM
// lanes (epilogue), warps 6..9 spread the nibbles, warp 10 stages scale codes.  Every wait is bounded; TMEM is
// freed on every exit path.
#include "mono_common.cuh"

extern void mono_set_error(const char* fmt, ...);

namespace mono {
namespace tc4bs {

constexpr int kThreads = 384;
constexpr int kUnit = 2;                // k tiles (128 elements) per staging slot: one 128-byte-wide box of nibbles
constexpr int kStages = 6;              // staging slots: 96 KB of packed weights in flight per SM
constexpr int kPackBytes = 128 * 128;   // a box of packed nibbles: 128 rows x 128 bytes = 256 k values per row
constexpr int kBBytes = 16 * 128;       // one k tile of activations (16 rows x 128 E4M3 bytes, 128-byte swizzle)
constexpr int kStageBytes = kPackBytes + kUnit * kBBytes;
constexpr int kABytes = 128 * 128;      // a padded operand tile: 128 rows x 128 bytes hold 128 x 128 nibbles
constexpr int kOpBytes = kUnit * (kABytes + kBBytes);  // an operand buffer: two weight tiles, then two activation tiles
constexpr int kOps = 2;
constexpr int kMaxSegTiles = 16;        // k tiles per segment
constexpr int kScSlots = 2;
constexpr int kSfBlock = 512;           // scale codes in the order tcgen05.cp wants
constexpr int kSfaBytes = kMaxSegTiles * kSfBlock;        // weights: a block per tile
constexpr int kSfbStep = 256;                             // activations: blocks half a block apart
constexpr int kSfbBytes = kMaxSegTiles * kSfbStep + kSfBlock / 2;
constexpr int kSlotBytes = kSfaBytes + kSfbBytes + 128;   // + the segment's coefficients
constexpr int kAccCols = 16;            // one accumulator: 16 columns (the step's rows); [2 segments in turn][2 issuers]
constexpr int kSfaCol = 4 * kAccCols;   // four sets of 4 weight-scale columns (two per issuer, in turn)
constexpr int kSfbCol = kSfaCol + 16;   // four sets of 4 activation-scale columns
constexpr int kTmemCols = 128;

struct Params {
    mono_gemv_args a;
};
MONO_TL_DECLARE(tl_bs)
#ifdef MONO_TIMELINE
// stamps of CTA 0's roles, units 32.. of the launch (steady state): row 150 + k, one column per unit
#define BS_TL(k, n) do { if (blockIdx.x == 0 && (n) >= 32 && (n) < 32 + MONO_TL_POINTS) tl_bs[150 + (k)][(n) - 32] = globaltimer_ns(); } while (0)
#else
#define BS_TL(k, n) do { } while (0)
#endif

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
// 32 lanes x 128 bits of shared memory to 4 TMEM columns, the same 32 rows in each of the four lane quarters
__device__ __forceinline__ void cp_sf(uint32_t tmem_col, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void mma_bs(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
// 16 TMEM columns (one accumulator) of this thread's lane
__device__ __forceinline__ void ld16(uint32_t taddr, uint32_t r[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
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
// Block-scaled descriptor: A E2M1 (format 5), B E4M3 (format 0), both K-major, N = 16, E8M0 scales, M = 128;
// group g of the tile: byte g of the scale columns for both operands
__device__ __forceinline__ uint32_t idesc_group(uint32_t g) {
    return (g << 4) | (5u << 7) | (0u << 10) | ((16u >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | (g << 29);
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1) gemv_tc4bs_kernel(const __grid_constant__ Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;                                    // kStages staging slots
    uint8_t* ops = ring + (size_t)kStages * kStageBytes;     // kOps operand buffers
    uint8_t* sc_ring = ops + (size_t)kOps * kOpBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sc_ring + (size_t)kScSlots * kSlotBytes);
    uint64_t* full = bars;                      // TMA -> converters: a slot's boxes have landed
    uint64_t* stage_free = full + kStages;      // 4 converter warps -> TMA: the slot has been spread
    uint64_t* op_full = stage_free + kStages;   // 4 converter warps -> MMA: an operand buffer is written
    uint64_t* op_free = op_full + kOps;         // MMA -> converters: the MMAs that read the buffer are done
    uint64_t* sc_full = op_free + kOps;         // scale warp -> MMA / epilogue: a segment's codes are staged
    uint64_t* sc_empty = sc_full + kScSlots;    // 2 issuers (their copies are done) + 4 epilogue warps (coefficients read)
    uint64_t* acc_full = sc_empty + kScSlots;   // 2 issuers -> epilogue: a segment's accumulators are complete
    uint64_t* acc_empty = acc_full + 2;         // 4 epilogue warps -> MMA
    __shared__ int abort_flag;
    __shared__ uint32_t tmem_base_s;
    __shared__ int s_elist[MONO_GEMV_MAX_JOBS][128];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rows = p.a.rows;
    if (tid == 0) {
        abort_flag = guard_failed(p.a.guard) ? 1 : 0;
        for (int i = 0; i < kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&stage_free[i], 4); }
        for (int i = 0; i < kOps; ++i) { mbar_init(&op_full[i], 4); mbar_init(&op_free[i], 1); }
        for (int i = 0; i < kScSlots; ++i) { mbar_init(&sc_full[i], 32); mbar_init(&sc_empty[i], 6); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 2); mbar_init(&acc_empty[i], 4); }
        mbar_fence_init();
    }
    // every code byte the MMA may look at holds a valid code from the start (2^0), whatever a segment fills in;
    // the padding halves of the operand buffers start at zero
    for (int i = tid; i < kScSlots * kSlotBytes / 4; i += kThreads) reinterpret_cast<uint32_t*>(sc_ring)[i] = 0x7F7F7F7Fu;
    for (int i = tid; i < kOps * kOpBytes / 16; i += kThreads) reinterpret_cast<uint4*>(ops)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_proxy_async_smem();
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

// every role walks the same (task, segment) sequence
#define BS_FOR_EACH_SEGMENT(...)                                                                                \
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
        // ------------------------------------------------------------ producer: packed weight boxes and activation tiles by TMA
        if (lane == 0) {
            int stage = 0, tl_n = 0;
            (void)tl_n;
            uint32_t phase = 0;
#define TASK_BEGIN
#define TASK_END
            BS_FOR_EACH_SEGMENT({
                const CUtensorMap* wmap = reinterpret_cast<const CUtensorMap*>(&jb.tmap);  // bytes: 128 per box row = 256 nibbles
                const CUtensorMap* amap = reinterpret_cast<const CUtensorMap*>(&jb.act_tmap);
                for (int t = 0; t < s.nt; t += kUnit) {
                    const int n2 = min(kUnit, s.nt - t);
                    if (!mbar_wait(&stage_free[stage], phase ^ 1, abortp, wait_ns)) break;
                    BS_TL(0, tl_n);
                    uint8_t* st = ring + (size_t)stage * kStageBytes;
                    // (a box that reaches past K reads zeros there and still counts its full size)
                    mbar_expect_tx(&full[stage], kPackBytes + n2 * kBBytes);
                    tma_load_3d(st, wmap, (s.t0 + t) * 64, s.row0, s.c2, &full[stage]);
                    for (int i = 0; i < n2; ++i)
                        tma_load_3d(st + kPackBytes + i * kBBytes, amap, (s.t0 + t + i) * 128, 0, s.aset, &full[stage]);
                    BS_TL(1, tl_n);
                    ++tl_n;
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            })
#undef TASK_BEGIN
#undef TASK_END
        }
    } else if (warp == 1 || warp == 11) {
        // ------------------------------------------------------------ scale copies + MMA: issuer `me` takes the launch's
        // units n = me, me + 2, ... (operand buffer `me`) and adds them into its own accumulator of the segment
        if (lane == 0) {
            const int me = warp == 1 ? 0 : 1;
            int slot = 0, buf = 0, n = 0, tl_n = 0;
            (void)tl_n;
            uint32_t ophase = 0, sphase = 0, aphase = 0, tile_no = 0;
#define TASK_BEGIN
#define TASK_END
            BS_FOR_EACH_SEGMENT({
                if (!mbar_wait(&sc_full[slot], sphase, abortp, wait_ns)) break;
                if (!mbar_wait(&acc_empty[buf], aphase ^ 1, abortp, wait_ns)) break;
                fence_after();
                const uint32_t sl = smem_u32(sc_ring + (size_t)slot * kSlotBytes);
                const uint32_t acc = tmem_base + (buf * 2 + me) * kAccCols;
                uint32_t accumulate = 0;
                for (int t = 0; t < s.nt; t += kUnit, ++n) {
                    if ((n & 1) != me) continue;
                    const int n2 = min(kUnit, s.nt - t);
                    if (me == 0) BS_TL(4, tl_n);
                    if (!mbar_wait(&op_full[me], ophase, abortp, wait_ns)) break;
                    if (me == 0) BS_TL(5, tl_n);
                    fence_after();
                    const uint32_t sa = smem_u32(ops + (size_t)me * kOpBytes);
                    for (int i = 0; i < n2; ++i) {
                        // the tile's codes to their TMEM columns (the tensor pipe runs a thread's copies and MMAs in the
                        // order it issued them; the column sets alternate all the same)
                        const int tt = t + i;
                        const uint32_t set = (me * 2 + (tile_no & 1)) * 4, sfa = tmem_base + kSfaCol + set, sfb = tmem_base + kSfbCol + set;
                        ++tile_no;
                        cp_sf(sfa, desc_sf(sl + tt * kSfBlock));
                        cp_sf(sfb, desc_sf(sl + kSfaBytes + tt * kSfbStep));
                        const uint64_t adesc = desc_sw128(sa + i * kABytes), bdesc = desc_sw128(sa + kUnit * kABytes + i * kBBytes);
#pragma unroll
                        for (uint32_t g = 0; g < 4; ++g) {  // one 32-value group per MMA, 32 bytes further along K
                            mma_bs(acc, adesc + 2 * g, bdesc + 2 * g, idesc_group(g), sfa, sfb, accumulate);
                            accumulate = 1;
                        }
                    }
                    commit(&op_free[me]);
                    if (me == 0) BS_TL(6, tl_n);
                    ++tl_n;
                    ophase ^= 1;
                }
                commit(&acc_full[buf]);
                commit(&sc_empty[slot]);
                if (++slot == kScSlots) { slot = 0; sphase ^= 1; }
                if (++buf == 2) { buf = 0; aphase ^= 1; }
            })
#undef TASK_BEGIN
#undef TASK_END
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue (TMEM lanes 32 * (warp % 4) ..)
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        const uint32_t tmem_lane = tmem_base + ((uint32_t)(q * 32) << 16);
        int slot = 0, buf = 0, n = 0;
        uint32_t sphase = 0, aphase = 0;
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
        BS_FOR_EACH_SEGMENT({
            if (!mbar_wait(&sc_full[slot], sphase, abortp, wait_ns)) break;
            if (!mbar_wait(&acc_full[buf], aphase, abortp, wait_ns)) break;
            fence_after();
            uint32_t d[32];
            ld32(tmem_lane + buf * 2 * kAccCols, d);
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            // which issuers had a unit of this segment (an accumulator nobody wrote holds an older segment's sum)
            const int units = (s.nt + kUnit - 1) / kUnit;
            const bool w0 = units >= 2 || (n & 1) == 0, w1 = units >= 2 || (n & 1) == 1;
            n += units;
            const float* coef = reinterpret_cast<const float*>(sc_ring + (size_t)slot * kSlotBytes + kSfaBytes + kSfbBytes);
#pragma unroll
            for (int c = 0; c < kMaxRows; ++c)
                if (c < rows)
                    total_acc[c] += ((w0 ? __uint_as_float(d[c]) : 0.f) + (w1 ? __uint_as_float(d[kAccCols + c]) : 0.f)) * (s.coef ? coef[c] : 1.f);
            __syncwarp();
            if (lane == 0) mbar_arrive(&sc_empty[slot]);
            if (++slot == kScSlots) { slot = 0; sphase ^= 1; }
            if (++buf == 2) { buf = 0; aphase ^= 1; }
        })
#undef TASK_BEGIN
#undef TASK_END
    } else if (warp < 10) {
        // ------------------------------------------------------------ converters: a staged box of nibbles -> two padded tiles
        const int ct = tid - 6 * 32;  // 0..127
        int stage = 0, ob = 0, tl_n = 0;
        (void)tl_n;
        uint32_t phase = 0, ophase = 0;
#define TASK_BEGIN
#define TASK_END
        BS_FOR_EACH_SEGMENT({
            bool ok = true;
            for (int t = 0; t < s.nt && ok; t += kUnit) {
                const int n2 = min(kUnit, s.nt - t);
                if (!mbar_wait(&full[stage], phase, abortp, wait_ns)) { ok = false; break; }
                if (ct == 0) BS_TL(2, tl_n);
                if (!mbar_wait(&op_free[ob], ophase ^ 1, abortp, wait_ns)) { ok = false; break; }
                if (ct == 0) BS_TL(3, tl_n);
                const uint32_t src = smem_u32(ring + (size_t)stage * kStageBytes), dst = smem_u32(ops + (size_t)ob * kOpBytes);
                // Weights.  The box row r holds 128 bytes = 16 pieces of 8 bytes (16 nibbles each) in 8 swizzled
                // 16-byte chunks; piece 2 j + h of the row is piece (2 j + h) % 8 of tile j / 4, and goes to the low
                // half of that tile's 16-byte chunk of the same number, at the operand's own swizzled place.
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int idx = it * 128 + ct, r = idx >> 3, j = idx & 7, x = r & 7;
                    const uint4 v = lds128(src + r * 128 + ((j ^ x) << 4));
                    const uint32_t d = dst + (j >> 2) * kABytes + r * 128;
                    const int c0 = (2 * j) & 7;
                    sts64(d + ((c0 ^ x) << 4), v.x, v.y);
                    sts64(d + (((c0 + 1) ^ x) << 4), v.z, v.w);
                }
                // Activations: the two tiles as they are (both places are 1024-byte aligned: the swizzle carries over)
                for (int o = ct * 16; o < n2 * kBBytes; o += 128 * 16) sts128(dst + kUnit * kABytes + o, lds128(src + kPackBytes + o));
                fence_proxy_async_smem();  // the MMA reads these bytes through the async proxy
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&stage_free[stage]);
                    mbar_arrive(&op_full[ob]);
                }
                if (ct == 0) BS_TL(7, tl_n);
                ++tl_n;
                if (++stage == kStages) { stage = 0; phase ^= 1; }
                if (++ob == kOps) { ob = 0; ophase ^= 1; }
            }
            if (!ok) break;
        })
#undef TASK_BEGIN
#undef TASK_END
    } else if (warp == 10) {
        // ------------------------------------------------------------ scale warp: a segment's codes, one segment ahead
        int slot = 0;
        uint32_t sphase = 0;
#define TASK_BEGIN
#define TASK_END
        BS_FOR_EACH_SEGMENT({
            int ok = 1;
            if (lane == 0) ok = mbar_wait(&sc_empty[slot], sphase ^ 1, abortp, wait_ns) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            uint8_t* sl = sc_ring + (size_t)slot * kSlotBytes;
            // weights: lane l holds rows l, l + 32, l + 64, l + 96 of the block (rows past the matrix repeat the last
            // one); their four words are the lane's 16 bytes of the tile's block.
            const int last_row = jb.n_rows - 1 - rb * 128;
            const uint8_t* wrow[4];
#pragma unroll
            for (int rr = 0; rr < 4; ++rr) wrow[rr] = s.wsc + (size_t)min(rr * 32 + lane, last_row) * jb.wscale_ld;
            {
                // all of the segment's loads are issued before the first is stored: one memory round trip per segment
                uint32_t w[kMaxSegTiles][4];
#pragma unroll
                for (int k = 0; k < kMaxSegTiles; ++k) {
                    const int t = min(k, s.nt - 1);
#pragma unroll
                    for (int rr = 0; rr < 4; ++rr) w[k][rr] = __ldg(reinterpret_cast<const uint32_t*>(wrow[rr] + t * 4));
                }
#pragma unroll
                for (int k = 0; k < kMaxSegTiles; ++k)
                    if (k < s.nt)
                        *reinterpret_cast<uint4*>(sl + (size_t)k * kSfBlock + lane * 16) = make_uint4(w[k][0], w[k][1], w[k][2], w[k][3]);
            }
            // activations: row c's four codes of tile t are the first four bytes of row c of the tile's block (rows
            // past the step: 2^0); lanes 0..15 take the even tiles, 16..31 the odd ones
            {
                const int c = lane & 15;
                const uint8_t* arow = s.asc + (size_t)min(c, rows - 1) * jb.ascale_ld;
                for (int t0 = lane >> 4; t0 < s.nt; t0 += 8) {
                    uint32_t a4[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) a4[k] = __ldg(reinterpret_cast<const uint32_t*>(arow + min(t0 + 2 * k, s.nt - 1) * 4));
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int t = t0 + 2 * k;
                        if (t < s.nt)
                            *reinterpret_cast<uint32_t*>(sl + kSfaBytes + (size_t)t * kSfbStep + c * 16) = c < rows ? a4[k] : 0x7F7F7F7Fu;
                    }
                }
            }
            if (s.coef && lane < rows) reinterpret_cast<float*>(sl + kSfaBytes + kSfbBytes)[lane] = __ldg(s.coef + lane);
            fence_proxy_async_smem();  // the copies to TMEM read these bytes through the async proxy
            mbar_arrive(&sc_full[slot]);
            if (++slot == kScSlots) { slot = 0; sphase ^= 1; }
        })
#undef TASK_BEGIN
#undef TASK_END
    }
#undef BS_FOR_EACH_SEGMENT
    fence_before();
    __syncthreads();
    if (abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before the CTA's memory goes
        if (tid == 0 && !guard_failed(p.a.guard)) guard_fail(p.a.guard, MONO_ERR_DEADLINE, 103);
    }
    if (warp == 1) {
        fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace tc4bs
}  // namespace mono

#ifdef MONO_TIMELINE
extern "C" int mono_timeline_read_tc4bs(unsigned long long* out, int* ctas, int* points) {
    *ctas = MONO_TL_CTAS;
    *points = MONO_TL_POINTS;
    return (int)cudaMemcpyFromSymbol(out, mono::tc4bs::tl_bs, sizeof(unsigned long long) * MONO_TL_CTAS * MONO_TL_POINTS);
}
#endif

// Launches the block-scaled MXFP4 kernel for an argument block that mono_gemv_launch has validated.
// Returns -100 when the block cannot take this path (the caller then tries the per-group kernel).
int mono_gemv_tc4bs_launch(const mono_gemv_args* a, long tasks, cudaStream_t st) {
    using namespace mono;
    for (int j = 0; j < a->njobs; ++j) {
        const mono_gemv_job& jb = a->job[j];
        const unsigned long long* w4 = reinterpret_cast<const unsigned long long*>(&jb.tmap4);
        const unsigned long long* wa = reinterpret_cast<const unsigned long long*>(&jb.act_tmap);
        const unsigned long long* wb = reinterpret_cast<const unsigned long long*>(&jb.tmap);
        unsigned long long any4 = 0, anya = 0, anyb = 0;
        for (int i = 0; i < 16; ++i) { any4 |= w4[i]; anya |= wa[i]; anyb |= wb[i]; }
        const int seg = jb.mode == MONO_JOB_EXPERT_DOWN ? jb.k_tiles : (jb.split_tiles < jb.k_tiles ? jb.split_tiles : jb.k_tiles);
        if (!any4 || !anya || !anyb || !jb.act_natural || jb.planes != 1 || jb.rb_per_mat != 0 || 2 * seg > tc4bs::kMaxSegTiles ||
            (jb.wscale_ld & 3) || (jb.ascale_ld & 3) || (reinterpret_cast<uintptr_t>(jb.wscale_e8) & 3) ||
            (reinterpret_cast<uintptr_t>(jb.ascale_e8) & 3) || (jb.wscale_mat_stride & 3) || (jb.ascale_seg_stride & 3))
            return -100;
    }
    tc4bs::Params p;
    p.a = *a;
    const size_t smem = 1024 + (size_t)tc4bs::kStages * tc4bs::kStageBytes + (size_t)tc4bs::kOps * tc4bs::kOpBytes +
                        (size_t)tc4bs::kScSlots * tc4bs::kSlotBytes + 512;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        cudaError_t e = cudaFuncSetAttribute(tc4bs::gemv_tc4bs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        mono::attr_done(attr_once);
    }
    int grid = a->max_ctas > 0 ? a->max_ctas : mono_sm_count();
    if (grid > tasks) grid = (int)tasks;
    if (grid < 1) grid = 1;
    cudaError_t e = launch_k(tc4bs::gemv_tc4bs_kernel, grid, tc4bs::kThreads, smem, st, p);
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}
