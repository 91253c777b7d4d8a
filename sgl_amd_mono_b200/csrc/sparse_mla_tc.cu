// Sparse MLA decode attention on 5th-generation tensor cores, for 64 or more local heads.
//
// Reference counterpart: the split stage of glm53/gfx950/kernel.py:3638-3973 (64 keys per split,
// split-local max and sum, p rounded to bf16 before P.V, bf16 partial accumulator); the merge stage
// (:3975-4075) stays the kernel of sparse_mla.cu.
//
// sm_100a design.  A task is (row, chunk of 64 selected keys) for ALL heads of the rank: the heads are the
// 128 TMEM lanes (M = 128), so a chunk's cache rows are fetched once per row instead of once per group of
// 16 heads.  Both contractions run as tcgen05.mma kind::f8f6f4 with f32 accumulators in tensor memory:
//   S[head][key]  = sum_d Q[head][d] K[key][d]      M 128, N 64,  K 576 (18 steps of 32)
//   O[head][dim]  = sum_k P[head][k] V[k][dim]      M 128, N 256 (twice), K 64 (2 steps of 32)
// The cache rows stay the E4M3 bytes they are stored as (one f32 power-of-two scale per key, applied to
// the scores as a column factor and folded into P for the second product), so nothing is widened.  The
// bf16 operands (queries; probabilities rounded to bf16 as the reference rounds them) are split exactly
// into two E4M3 planes (value = (hi + lo) * 2^e with one exponent per head), the same split the FP8 GEMVs
// use for their bf16 activations.  A chunk is staged once, as 128-byte-swizzled blocks of [64 keys][128
// dims]: read K-major they are the B operand of the first product, read MN-major (keys as the contraction
// dimension) they are the B operand of the second, so no transposed copy is made.
//
// The query planes of a row are prepared once per launch by mla_qsplit_kernel as an image of the shared
// memory operand (swizzle applied), which every task of the row fetches with bulk copies.
#include "mono_common.cuh"

extern void mono_set_error(const char* fmt, ...);

namespace mla_tc {
using namespace mono;
MONO_TL_DECLARE(tl_split)

constexpr int kThreads = 256;
constexpr int kKeys = 64;                        // keys per task
constexpr int kBlocks = 5;                       // 128-dim column blocks of a 576-dim row (the last holds 64)
constexpr int kQBlockBytes = 128 * 128;          // [128 heads][128 B]
constexpr int kQPlaneBytes = kBlocks * kQBlockBytes;
constexpr int kQBytes = 2 * kQPlaneBytes;        // hi and lo planes
constexpr int kKvBlockBytes = kKeys * 128;       // [64 keys][128 B]
constexpr int kKvBytes = kBlocks * kKvBlockBytes;
constexpr int kRowImage = kQBytes + 128 * 4;     // the planes, then one f32 scale per head
constexpr int kStagePitch = 80;                  // bytes per staged row of 32 bf16 values: conflict-free 16-byte accesses
constexpr int kStageBytes = 8 * 32 * kStagePitch;  // one tile of 32 heads x 32 columns per warp
constexpr int kSmemBytes = 1024 + kQBytes + kKvBytes + kStageBytes;
constexpr int kTmemCols = 512;

// ---- tcgen05 wrappers (one CTA per MMA group)
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 32 columns of f32: thread t of the warp gets lane t's columns
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t r[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptors, 128-byte swizzle, version 1 (sm_100).  K-major: rows of 128 bytes, groups
// of eight rows `sbo` bytes apart.  MN-major: atoms of 128 contiguous bytes x 8 contraction rows; atoms `sbo`
// bytes apart along the contraction dimension and `lbo` bytes apart along the other.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptors: D f32, A and B E4M3, M = 128.
constexpr uint32_t kIdescS = (1u << 4) | ((64u >> 3) << 17) | ((128u >> 4) << 24);                   // N 64, both K-major
constexpr uint32_t kIdescPV = (1u << 4) | (1u << 16) | ((256u >> 3) << 17) | ((128u >> 4) << 24);    // N 256, B MN-major

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// 16 bf16 values -> 16 hi bytes and 16 lo bytes of (value * inv): value * inv = hi + lo exactly for values within
// 2^12 of the largest (E4M3 carries four significant bits, a bf16 eight)
__device__ __forceinline__ void split16(const float v[16], float inv, uint4* hi, uint4* lo) {
    uint32_t h[4] = {0, 0, 0, 0}, l[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        const float2 sv = make_float2(v[i] * inv, v[i + 1] * inv);
        const __nv_fp8x2_storage_t hb = __nv_cvt_float2_to_fp8x2(sv, __NV_SATFINITE, __NV_E4M3);
        const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(hb, __NV_E4M3);
        const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&hr));
        const __nv_fp8x2_storage_t lb = __nv_cvt_float2_to_fp8x2(make_float2(sv.x - hf.x, sv.y - hf.y), __NV_SATFINITE, __NV_E4M3);
        h[i >> 2] |= (uint32_t)hb << (8 * (i & 3));
        l[i >> 2] |= (uint32_t)lb << (8 * (i & 3));
    }
    *hi = make_uint4(h[0], h[1], h[2], h[3]);
    *lo = make_uint4(l[0], l[1], l[2], l[3]);
}

// One warp per head: the head's 576 bf16 query values -> two E4M3 planes in the layout the first product's A
// operand has in shared memory (five blocks of [128 heads][128 bytes], 16-byte pieces XOR-swizzled by the head's
// low three bits), and the head's power-of-two scale.  Heads past a.heads get zero planes.
__global__ void __launch_bounds__(128) mla_qsplit_kernel(const mono_sparse_mla_args a, uint8_t* image) {
    pdl_prologue();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x >> 5, head = (blockIdx.x & 31) * 4 + warp;
    uint8_t* img = image + (size_t)row * kRowImage;
    const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(a.q) + ((size_t)row * a.heads + head) * kKvDim;
    // piece p (16 values) of the row: lane handles piece `lane`, lanes 0..3 also piece 32 + lane
    float v[2][16];
    float amax = 0.f;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int piece = t * 32 + lane;
        const bool live = head < a.heads && piece < kKvDim / 16;
#pragma unroll
        for (int i = 0; i < 16; i += 8) {
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (live) raw = *reinterpret_cast<const uint4*>(q + piece * 16 + i);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
                v[t][i + 2 * j] = f.x;
                v[t][i + 2 * j + 1] = f.y;
                amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
        }
    }
    amax = warp_max(amax);
    const int code = code_ceil(fmaxf(amax, 7.888609052210118e-31f /* 2^-100 */) / 448.f);
    const float inv = exp2_code(254 - code);
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int piece = t * 32 + lane;
        if (piece < kKvDim / 16) {
            uint4 hi, lo;
            split16(v[t], inv, &hi, &lo);
            const int blk = piece >> 3, c = piece & 7;
            uint8_t* dst = img + blk * kQBlockBytes + head * 128 + ((c ^ (head & 7)) << 4);
            *reinterpret_cast<uint4*>(dst) = hi;
            *reinterpret_cast<uint4*>(dst + kQPlaneBytes) = lo;
        }
    }
    if (lane == 0) reinterpret_cast<float*>(img + kQBytes)[head] = exp2_code(code);
}

__global__ void __launch_bounds__(kThreads, 1) sparse_mla_split_tc_kernel(const mono_sparse_mla_args a, const uint8_t* image, int nchunks) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* qbuf = smem;             // the query planes; the probability planes reuse its first 32 KB
    uint8_t* kvbuf = smem + kQBytes;  // the chunk's cache rows
    uint8_t* stage = kvbuf + kKvBytes;  // the epilogue's transposition tiles
    __shared__ float s_kscale[kKeys], s_qscale[128], s_prow[128], s_x[2][128];
    __shared__ int s_slot[kKeys];
    __shared__ uint64_t bar_q, bar_mma;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int* abortp = &abort_flag;
    if (tid == 0) {
        abort_flag = guard_failed(a.guard) ? 1 : 0;
        mbar_init(&bar_q, 1);
        mbar_init(&bar_mma, 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&tmem_base_s, kTmemCols);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_launch_dependents();
    pdl_wait();
    __nv_bfloat16* part_acc = reinterpret_cast<__nv_bfloat16*>(a.scratch);
    float* part_ml = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a.scratch) +
                                              (size_t)a.rows * nchunks * a.heads * 512 * sizeof(__nv_bfloat16));
    const uint32_t q_addr = smem_u32(qbuf), kv_addr = smem_u32(kvbuf);
    uint32_t qph = 0, mph = 0;
    const int total = a.rows * nchunks;
    // A CTA takes a contiguous run of tasks (chunks of one row, mostly): the row's query planes stay in shared
    // memory from one chunk to the next, and only the 32 KB the probability planes overwrote are fetched again.
    const int t0 = (int)((long)blockIdx.x * total / gridDim.x), t1 = (int)((long)(blockIdx.x + 1) * total / gridDim.x);
    // Requests what `task` needs (query planes or the part of them that was overwritten, the chunk's slots and key
    // scales, the chunk's cache rows) without waiting for any of it; `have_row` is the row whose planes are resident.
    // a chunk's slot and key scale for thread tid < 64 (two dependent loads: asked for a task ahead)
    auto slot_of = [&](int task, int* slot_out, float* scale_out) {
        const int row = task / nchunks, chunk = task - row * nchunks;
        const int kidx = chunk * kKeys + tid;
        int slot = kidx < a.topk ? a.topk_slots[(size_t)row * a.topk_ld + kidx] : -1;
        if (slot >= 0 && (int64_t)slot >= a.n_pages * kPage) slot = -1;
        float sc = 0.f;
        if (slot >= 0) sc = __ldg(reinterpret_cast<const float*>(a.kv_pages + (size_t)(slot / kPage) * kKvPageBytes + kPage * kKvDim) + slot % kPage);
        *slot_out = slot;
        *scale_out = sc;
    };
    int pre_slot = -1;
    float pre_scale = 0.f;
    auto request = [&](int task, int have_row) -> bool {
        const int row = task / nchunks;
        const bool full = row != have_row;
        if (tid == 0) {
            const uint8_t* src = image + (size_t)row * kRowImage;
            const int nblk = full ? kQBytes / kQBlockBytes : 2;
            mbar_expect_tx(&bar_q, nblk * kQBlockBytes);
#pragma unroll 1
            for (int i = 0; i < nblk; ++i) bulk_load(qbuf + i * kQBlockBytes, src + (size_t)i * kQBlockBytes, kQBlockBytes, &bar_q);
        }
        if (tid < kKeys) {
            s_slot[tid] = pre_slot;
            s_kscale[tid] = pre_scale;
        } else if (tid >= 128 && full) {
            s_qscale[tid - 128] = reinterpret_cast<const float*>(image + (size_t)row * kRowImage + kQBytes)[tid - 128];
        }
        __syncthreads();
        // gather: 64 keys x 36 sixteen-byte pieces, each to its swizzled place; every copy is in flight at once
        constexpr int kPieces = kKvDim / 16;                  // 36
        constexpr int kPer = kKeys * kPieces / kThreads;      // 9
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int c = tid + i * kThreads;
            const int key = c / kPieces, piece = c - key * kPieces;
            const int slot = s_slot[key];
            const uint32_t dst = kv_addr + (piece >> 3) * kKvBlockBytes + key * 128 + (((piece & 7) ^ (key & 7)) << 4);
            if (slot >= 0) {
                cp_async16(dst, a.kv_pages + (size_t)(slot / kPage) * kKvPageBytes + (size_t)(slot % kPage) * kKvDim + piece * 16);
            } else {
                asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0u) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        return true;
    };
    MONO_TL(tl_split, 0);
    if (t0 < t1 && tid < kKeys) slot_of(t0, &pre_slot, &pre_scale);
    if (t0 < t1 && !*abortp) request(t0, -1);
    for (int task = t0; task < t1 && !*abortp; ++task) {
        const int row = task / nchunks, chunk = task - row * nchunks;
        const int tl = 1 + 6 * (task - t0);  // timeline points of this task (the first two tasks fit)
        // ---- this task's operands have been requested: wait for them
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these writes before the tensor core's reads
        if (!mbar_wait(&bar_q, qph, abortp)) break;
        qph ^= 1;
        __syncthreads();
        if (task + 1 < t1 && tid < kKeys) slot_of(task + 1, &pre_slot, &pre_scale);  // in flight during this task's products
        MONO_TL(tl_split, tl);
        // ---- S = Q K^T: hi and lo planes, five blocks, 32 bytes of the contraction per MMA
        if (tid == 0) {
            fence_after();
            // the hi and the lo plane accumulate in columns 0..63 and 64..127: two independent chains of MMAs
            uint32_t acc = 0;
#pragma unroll 1
            for (int blk = 0; blk < kBlocks; ++blk) {
                const uint64_t ah = desc_sw128(q_addr + blk * kQBlockBytes, 0, 1024);
                const uint64_t al = desc_sw128(q_addr + kQPlaneBytes + blk * kQBlockBytes, 0, 1024);
                const uint64_t bd = desc_sw128(kv_addr + blk * kKvBlockBytes, 0, 1024);
                const int steps = blk < 4 ? 4 : 2;
                for (int k = 0; k < steps; ++k) {
                    mma_f8(tmem_base, ah + 2 * k, bd + 2 * k, kIdescS, acc);
                    mma_f8(tmem_base + 64, al + 2 * k, bd + 2 * k, kIdescS, acc);
                    acc = 1;
                }
            }
            mma_commit(&bar_mma);
        }
        if (!mbar_wait(&bar_mma, mph, abortp)) break;
        mph ^= 1;
        fence_after();
        MONO_TL(tl_split, tl + 1);
        // ---- softmax over the chunk: head = TMEM lane; warps w and w + 4 share a lane quarter and take 32 keys each
        {
            const int head = (warp & 3) * 32 + lane, kh = warp >> 2;  // kh: which half of the keys
            uint32_t raw[32], raw_lo[32];
            float s[32];
            const float qs = s_qscale[head] * a.sm_scale;
            tmem_ld32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + kh * 32, raw);
            tmem_ld32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + 64 + kh * 32, raw_lo);
            float mloc = -INFINITY;
#pragma unroll
            for (int k = 0; k < 32; ++k) {
                const int key = kh * 32 + k;
                s[k] = s_slot[key] >= 0 ? (__uint_as_float(raw[k]) + __uint_as_float(raw_lo[k])) * (qs * s_kscale[key]) : -INFINITY;
                mloc = fmaxf(mloc, s[k]);
            }
            s_x[kh][head] = mloc;
            __syncthreads();
            const float m = fmaxf(s_x[0][head], s_x[1][head]);
            float l = 0.f, amax = 0.f;
#pragma unroll
            for (int k = 0; k < 32; ++k) {
                const float p = (m == -INFINITY) ? 0.f : __expf(s[k] - m);
                l += p;
                // the probability as the reference feeds it to P.V (rounded to bf16), times the key's scale
                s[k] = bf16_round(p) * s_kscale[kh * 32 + k];
                amax = fmaxf(amax, s[k]);
            }
            __syncthreads();  // both halves have read the maxima
            s_x[kh][head] = amax;
            if (kh == 1) s_prow[head] = l;  // the upper half's sum, on its way to the lower half's thread
            __syncthreads();
            amax = fmaxf(s_x[0][head], s_x[1][head]);
            const int code = code_ceil(fmaxf(amax, 7.888609052210118e-31f) / 448.f);
            const float inv = exp2_code(254 - code);
            if (kh == 0) l += s_prow[head];
            __syncthreads();  // the sums have been taken before the slot gets the row's scale
            if (kh == 0) s_prow[head] = exp2_code(code);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint4 hi, lo;
                split16(&s[c * 16], inv, &hi, &lo);
                const uint32_t dst = q_addr + head * 128 + (((kh * 2 + c) ^ (head & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + kQBlockBytes), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w) : "memory");
            }
            if (kh == 0 && head < a.heads) {
                float* ml = part_ml + (((size_t)row * nchunks + chunk) * a.heads + head) * 2;
                ml[0] = m;
                ml[1] = l;
            }
        }
        fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        MONO_TL(tl_split, tl + 2);
        // ---- O = P V: two halves of 256 latent dims, hi and lo planes, two steps of 32 keys
        if (tid == 0) {
            fence_after();
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                uint32_t acc = 0;
#pragma unroll 1
                for (int pl = 0; pl < 2; ++pl) {
                    const uint64_t ad = desc_sw128(q_addr + pl * kQBlockBytes, 0, 1024);
                    for (int ks = 0; ks < 2; ++ks) {
                        // keys 32 ks .. of column blocks 2 half, 2 half + 1: atoms of 8 keys 1024 B apart, blocks 8192 B apart
                        const uint64_t bd = desc_sw128(kv_addr + 2 * half * kKvBlockBytes + ks * 32 * 128, kKvBlockBytes, 1024);
                        mma_f8(tmem_base + half * 256, ad + 2 * ks, bd, kIdescPV, acc);
                        acc = 1;
                    }
                }
            }
            mma_commit(&bar_mma);
        }
        if (!mbar_wait(&bar_mma, mph, abortp)) break;
        mph ^= 1;
        fence_after();
        MONO_TL(tl_split, tl + 3);
        // both products are done with shared memory: the next task's operands travel during this task's epilogue
        if (task + 1 < t1) request(task + 1, row);
        MONO_TL(tl_split, tl + 4);
        // ---- the task's partial: warp w holds lanes 32 (w % 4) .., columns 256 (w / 4) ..  A thread's 32 columns of a
        // head are 64 bytes of that head's row; the warp transposes its 32 x 64 B tile through shared memory so that four
        // lanes write one head's 64 bytes together (eight full half-lines per store instead of 32 quarter-filled sectors)
        {
            const int hq = (warp & 3) * 32, col0 = (warp >> 2) * 256;
            const float sc = s_prow[hq + lane];
            uint8_t* tile = stage + warp * 32 * kStagePitch;
            __nv_bfloat16* dst0 = part_acc + (((size_t)row * nchunks + chunk) * a.heads + hq) * 512 + col0;
#pragma unroll 1
            for (int c = 0; c < 256; c += 32) {
                uint32_t raw[32];
                tmem_ld32(tmem_base + ((uint32_t)hq << 16) + col0 + c, raw);
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(raw[i + 2 * j]) * sc, __uint_as_float(raw[i + 2 * j + 1]) * sc);
                        w[j] = *reinterpret_cast<const uint32_t*>(&b);
                    }
                    *reinterpret_cast<uint4*>(tile + lane * kStagePitch + i * 2) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                __syncwarp();
#pragma unroll
                for (int pass = 0; pass < 4; ++pass) {
                    const int r = pass * 8 + (lane >> 2), piece = lane & 3;
                    const uint4 v = *reinterpret_cast<const uint4*>(tile + r * kStagePitch + piece * 16);
                    if (hq + r < a.heads) *reinterpret_cast<uint4*>(dst0 + (size_t)r * 512 + c + piece * 8) = v;
                }
                __syncwarp();
            }
        }
        fence_before();
        __syncthreads();  // tensor memory and both buffers are free for the next task
        MONO_TL(tl_split, tl + 5);
    }
    fence_before();
    __syncthreads();
    if (*abortp) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before the CTA's memory goes
        if (tid == 0 && !guard_failed(a.guard)) guard_fail(a.guard, MONO_ERR_DEADLINE, 102);
    }
    if (warp == 0) {
        fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace mla_tc

// Bytes of query image a launch of `rows` rows needs behind the split partials.
size_t mono_sparse_mla_tc_image_bytes(int rows) { return (size_t)rows * mla_tc::kRowImage + 1024; }

// Prepares the query planes and runs the tcgen05 split for a validated argument block; the partials have the
// layout of the warp-MMA split with nsplit = nchunks, so the merge kernel of sparse_mla.cu follows unchanged.
int mono_sparse_mla_tc_split(const mono_sparse_mla_args* a, int nchunks, cudaStream_t st) {
    using namespace mla_tc;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        const cudaError_t e = cudaFuncSetAttribute(sparse_mla_split_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) {
            mono_set_error("mono_sparse_mla_launch: %s", cudaGetErrorString(e));
            return (int)e;
        }
        mono::attr_done(attr_once);
    }
    const size_t part = (size_t)a->rows * nchunks * a->heads * (512 * sizeof(__nv_bfloat16) + 2 * sizeof(float));
    uint8_t* image = reinterpret_cast<uint8_t*>(a->scratch) + ((part + 1023) & ~size_t(1023));
    mono::launch_k(mla_qsplit_kernel, a->rows * 32, 128, 0, st, *a, image);
    const int sms = mono_sm_count();
    int grid = a->rows * nchunks;
    if (grid > sms) grid = sms;
    mono::launch_k(sparse_mla_split_tc_kernel, grid, kThreads, kSmemBytes, st, *a, (const uint8_t*)image, nchunks);
    return 0;
}

#ifdef MONO_TIMELINE
// Copies the split kernel's stamps of the last launch to `out` (MONO_TL_CTAS x MONO_TL_POINTS); blocks the host.
extern "C" int mono_timeline_read_mla_split(unsigned long long* out, int* ctas, int* points) {
    *ctas = MONO_TL_CTAS;
    *points = MONO_TL_POINTS;
    return (int)cudaMemcpyFromSymbol(out, mla_tc::tl_split, sizeof(unsigned long long) * MONO_TL_CTAS * MONO_TL_POINTS);
}
#endif
