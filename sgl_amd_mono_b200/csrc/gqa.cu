// GQA block-sparse decode attention: head norms + RoPE + cache insert, block scores, exact
// top-16 block selection, attention over the selected blocks (split + merge).
//
// Reference counterparts (sgl_amd_mono/minimax_m3/gfx950): pre_attn.py:8-19 (per-head Gemma
// RMSNorm, partial NeoX RoPE, K / V to the FP8 cache with the layer's fixed scale, index key as
// E4M3 with unit scale), index_score.py:1-12 (block score = max over causal keys of
// index_q . index_k times fp32(sm_scale * log2 e)), post_attn.py:466-592 with select.py:1-56
// (pinned init / local blocks, rank by counting (key, block id) descending, tail block last),
// post_attn.py:706-979 (split-local softmax and merge).  A block is one 64-token page.
#include "mono_common.cuh"

extern void mono_set_error(const char* fmt, ...);

namespace mono {

constexpr int kGqaDim = 128;
constexpr int kGqaBlock = 64;
constexpr int kGqaTopk = 16;
constexpr int kGqaMaxGroup = 8;

// ------------------------------------------------------------------ front
// grid (rows, q_heads + 2 * kv_heads + 2), 128 threads: one head each
__global__ void __launch_bounds__(kGqaDim, 4) gqa_front_kernel(const mono_gqa_args a) {
    pdl_prologue();
    __shared__ float red[4];
    __shared__ float y[kGqaDim];
    const int row = blockIdx.x, hh = blockIdx.y, tid = threadIdx.x;
    const int nq = a.q_heads, nk = a.kv_heads;
    // 0: q, 1: k, 2: v, 3: index q, 4: index k
    const int kind = hh < nq ? 0 : hh < nq + nk ? 1 : hh < nq + 2 * nk ? 2 : hh == nq + 2 * nk ? 3 : 4;
    const int64_t slot = a.slots ? a.slots[row] : 0;
    if (slot < 0 && (kind == 1 || kind == 2 || kind == 4)) return;  // a pad row inserts nothing
    float x = 0.f;
    const float* src = a.qkv + (size_t)row * a.ld + hh * kGqaDim + tid;
#pragma unroll 4
    for (int s = 0; s < a.nsum; ++s) x += src[(size_t)s * a.sum_stride];
    float v = x;
    if (kind != 2) {
        float ssq = warp_sum(x * x);
        if ((tid & 31) == 0) red[tid >> 5] = ssq;
        __syncthreads();
        const float tot = red[0] + red[1] + red[2] + red[3];
        const float rstd = rsqrtf(tot / (float)kGqaDim + a.eps);
        const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(kind == 0 ? a.g_q : kind == 1 ? a.g_k : kind == 3 ? a.g_iq : a.g_ik);
        v = bf16_round(x * rstd * (1.f + __bfloat162float(g[tid])));
        y[tid] = v;
        __syncthreads();
        if (tid < 64) {
            const int64_t pos = a.positions[row];
            const int i = tid & 31;
            const float c = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.cos)[pos * 32 + i]);
            const float s = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.sin)[pos * 32 + i]);
            const float lo = y[i], hi = y[i + 32];
            v = tid < 32 ? bf16_round(lo * c - hi * s) : bf16_round(hi * c + lo * s);
        }
    } else {
        v = bf16_round(x);
    }
    if (kind == 0) {
        reinterpret_cast<__nv_bfloat16*>(a.q_out)[((size_t)row * nq + hh) * kGqaDim + tid] = __float2bfloat16_rn(v);
    } else if (kind == 3) {
        reinterpret_cast<__nv_bfloat16*>(a.iq_out)[(size_t)row * kGqaDim + tid] = __float2bfloat16_rn(v);
    } else if (slot < a.n_pages * kGqaBlock) {
        if (kind == 4) {
            a.index_cache[(size_t)slot * kGqaDim + tid] = f32_to_e4m3(v);
        } else {
            const int h = kind == 1 ? hh - nq : hh - nq - nk;
            const float sc = kind == 1 ? a.k_scale : a.v_scale;
            uint8_t* cache = kind == 1 ? a.k_cache : a.v_cache;
            cache[((size_t)slot * nk + h) * kGqaDim + tid] = f32_to_e4m3(fminf(fmaxf(__fdiv_rn(v, sc), -448.f), 448.f));
        }
    }
}

// ------------------------------------------------------------------ block scores
// grid (rows * ceil(score_ld / 4)), 256 threads: four blocks per CTA, two warps per block; the row's index
// query is staged once per CTA
constexpr int kScoreBlocksPerCta = 4;

__global__ void __launch_bounds__(kGqaBlock * kScoreBlocksPerCta) gqa_score_kernel(const mono_gqa_args a, float scale) {
    pdl_prologue();
    __shared__ __align__(16) float q[kGqaDim];
    __shared__ float red[2 * kScoreBlocksPerCta];
    const int groups = (a.score_ld + kScoreBlocksPerCta - 1) / kScoreBlocksPerCta;
    const int row = blockIdx.x / groups, tid = threadIdx.x;
    const int sub = tid >> 6, key = tid & 63;
    const int b = (blockIdx.x - row * groups) * kScoreBlocksPerCta + sub;
    // The slot, the position and the page number are asked for together, and the block's keys as soon as the page
    // number is known: two memory round trips before the arithmetic instead of four (the query is staged while the
    // keys are in flight).  Every load is unconditional, from a clamped address.
    const int slot_v = a.slots ? (int)a.slots[row] : 0;
    const int seq = (int)a.positions[row] + 1;
    const int b_ld = min(b, a.score_ld - 1);
    const int page_raw = a.page_table[(size_t)row * a.pt_ld + b_ld];
    const __nv_bfloat16* iq = reinterpret_cast<const __nv_bfloat16*>(a.iq_out) + (size_t)row * kGqaDim;
    const float qv_stage = tid < kGqaDim ? __bfloat162float(iq[tid]) : 0.f;
    const int lane = tid & 31, chunk = lane & 7, half = (tid >> 5) & 1;
    const bool page_ok = page_raw >= 0 && page_raw < a.n_pages;
    const uint8_t* base = a.index_cache + (size_t)(page_ok ? page_raw : 0) * kGqaBlock * kGqaDim;
    uint4 w[8];
#pragma unroll
    for (int it = 0; it < 8; ++it)
        w[it] = *reinterpret_cast<const uint4*>(base + (size_t)(half * 32 + it * 4 + (lane >> 3)) * kGqaDim + chunk * 16);
    if (slot_v < 0) return;
    const int n_blk = (seq + kGqaBlock - 1) / kGqaBlock;
    if ((b - sub) >= n_blk) return;  // the whole CTA is past the row's context
    if (tid < kGqaDim) q[tid] = qv_stage;
    __syncthreads();
    // eight lanes share a key row (16 bytes each: one coalesced 512-byte request covers four rows), so a warp
    // walks its 32 keys four at a time; the eight partial dots of a row meet in a 3-step butterfly
    float dot = -INFINITY;
    if (b < n_blk && b < a.score_ld) {
        if (page_ok) {
            const float4* q4 = reinterpret_cast<const float4*>(q) + chunk * 4;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const uint32_t ws[4] = {w[it].x, w[it].y, w[it].z, w[it].w};
                float d = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(ws[j] & 0xFFFFu), __NV_E4M3);
                    const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(ws[j] >> 16), __NV_E4M3);
                    const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
                    const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
                    const float4 qv = q4[j];
                    d += f01.x * qv.x;
                    d += f01.y * qv.y;
                    d += f23.x * qv.z;
                    d += f23.y * qv.w;
                }
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                const int k = half * 32 + it * 4 + (lane >> 3);
                if (b * kGqaBlock + k < seq) dot = fmaxf(dot, d);
            }
        }
    }
    const float m = warp_max(dot);
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();
    if (key == 0 && b < n_blk && b < a.score_ld) a.scores[(size_t)row * a.score_ld + b] = fmaxf(red[2 * sub], red[2 * sub + 1]) * scale;
}

// ------------------------------------------------------------------ selection
constexpr int kSelThreads = 1024;
constexpr int kSelMaxBlocks = 4096;

__device__ __forceinline__ int gqa_index_key(float sc, int b, int n_blk, int init_blocks, int local_blocks) {
    if (b < init_blocks) sc = 1e30f;
    if (b >= n_blk - local_blocks) sc = 1e29f;
    int bits = __float_as_int(sc);
    if (bits == (int)0x80000000) bits = 0;
    int key = bits < 0 ? bits ^ 0x7FFFFFFF : bits;
    if ((bits & 0x7FFFFFFF) > 0x7F800000) key = (int)0x80000000;
    return key;
}

__global__ void __launch_bounds__(kSelThreads, 1) gqa_select_kernel(const mono_gqa_args a) {
    pdl_prologue();
    extern __shared__ long long keys[];  // (key32 << 32) | block id
    __shared__ int s_tail_sel;
    const int row = blockIdx.x, tid = threadIdx.x;
    int32_t* out_b = a.sel_blocks + row * kGqaTopk;
    int32_t* out_p = a.sel_pages + row * kGqaTopk;
    if (tid < kGqaTopk) { out_b[tid] = -1; out_p[tid] = -1; }
    if (tid == 0) s_tail_sel = 0;
    if (a.slots && a.slots[row] < 0) {
        if (tid == 0) a.n_ctx[row] = 0;
        return;
    }
    const int seq = (int)a.positions[row] + 1;
    const int n_blk = min((seq + kGqaBlock - 1) / kGqaBlock, kSelMaxBlocks);
    const bool scored = n_blk > kGqaTopk;
    for (int b = tid; b < n_blk; b += kSelThreads) {
        const int key = scored ? gqa_index_key(a.scores[(size_t)row * a.score_ld + b], b, n_blk, a.init_blocks, a.local_blocks) : -b;
        keys[b] = ((long long)key << 32) | (long long)(unsigned)b;
    }
    __syncthreads();
    const int n_sel = min(n_blk, kGqaTopk), tail = n_blk - 1;
    const long long kt = keys[tail];
    // A floor under the 16th largest key: the 16th largest of the 32 warps' maxima (32 distinct entries are
    // at least their warp's maximum ... at least the 16th largest of those).  Only entries at or above the
    // floor can rank among the first 16, and every entry that beats one of them is itself above the floor:
    // ranks counted among those candidates are exact (select.py:57-101 group_floor / compact).
    __shared__ long long s_wmax[kSelThreads / 32];
    __shared__ long long s_floor;
    __shared__ int s_ncand;
    long long* cand = keys + kSelMaxBlocks;  // candidate list (dynamic shared memory after the keys)
    {
        long long mx = (long long)0x8000000000000000ll;
        for (int b = tid; b < n_blk; b += kSelThreads) mx = keys[b] > mx ? keys[b] : mx;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const long long other = __shfl_xor_sync(0xffffffffu, mx, o);
            mx = other > mx ? other : mx;
        }
        if ((tid & 31) == 0) s_wmax[tid >> 5] = mx;
        if (tid == 0) s_ncand = 0;
    }
    __syncthreads();
    if (tid < 32) {
        const long long mine = s_wmax[tid];
        int beaten = 0;
        for (int j = 0; j < 32; ++j) beaten += s_wmax[j] > mine || (s_wmax[j] == mine && j < tid);
        if (beaten == kGqaTopk - 1) s_floor = mine;  // the 16th largest warp maximum
    }
    __syncthreads();
    const long long floor_key = n_blk > kGqaTopk * 2 ? s_floor : (long long)0x8000000000000000ll;
    for (int b = tid; b < n_blk; b += kSelThreads)
        if (keys[b] >= floor_key) cand[atomicAdd(&s_ncand, 1)] = keys[b];
    __syncthreads();
    const int n_cand = s_ncand;
    int my_rank[kSelMaxBlocks / kSelThreads];
#pragma unroll
    for (int i = 0; i < kSelMaxBlocks / kSelThreads; ++i) {
        const int b = tid + i * kSelThreads;
        my_rank[i] = 1 << 30;
        if (b < n_blk && keys[b] >= floor_key) {
            const long long mine = keys[b];
            int r = 0;
            for (int j = 0; j < n_cand; ++j) r += cand[j] > mine;
            my_rank[i] = r;
            if (b == tail && r < n_sel) s_tail_sel = 1;
        }
    }
    __syncthreads();
    const int tail_sel = s_tail_sel;
    const int n_full = n_sel - tail_sel;
#pragma unroll
    for (int i = 0; i < kSelMaxBlocks / kSelThreads; ++i) {
        const int b = tid + i * kSelThreads;
        if (b < n_blk && my_rank[i] < n_sel) {
            const int slot = b == tail ? n_full : my_rank[i] - (kt > keys[b] ? 1 : 0);
            out_b[slot] = b;
            out_p[slot] = a.page_table[(size_t)row * a.pt_ld + b];
        }
    }
    if (tid == 0)
        a.n_ctx[row] = tail_sel ? n_full * kGqaBlock + seq - tail * kGqaBlock : min(n_sel * kGqaBlock, seq);
}

// ------------------------------------------------------------------ attention: split
// grid (rows * kv_heads * 16 slots), 128 threads.  Partial of one (row, kv head, slot):
// per q head of the group: m, l, acc[128].
struct GqaSplitSmem {
    float k[kGqaBlock][kGqaDim + 1];
    uint8_t v[kGqaBlock][kGqaDim];  // E4M3 bytes
    float q[kGqaMaxGroup][kGqaDim];
    float p[kGqaMaxGroup][kGqaBlock];
};

__global__ void __launch_bounds__(kGqaDim, 4) gqa_split_kernel(const mono_gqa_args a) {
    pdl_prologue();
    extern __shared__ uint8_t smem_raw[];
    GqaSplitSmem& sm = *reinterpret_cast<GqaSplitSmem*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slot = blockIdx.x % kGqaTopk, kvh = (blockIdx.x / kGqaTopk) % a.kv_heads, row = blockIdx.x / (kGqaTopk * a.kv_heads);
    const int G = a.q_heads / a.kv_heads;
    float* part = a.scratch + ((size_t)(row * a.kv_heads + kvh) * kGqaTopk + slot) * G * (kGqaDim + 2);
    const int n_ctx = a.n_ctx[row];
    const int page = a.sel_pages[row * kGqaTopk + slot];
    const int live = min(kGqaBlock, n_ctx - slot * kGqaBlock);
    if (page < 0 || page >= a.n_pages || live <= 0) {
        for (int g = warp; g < G; g += 4)
            if (lane == 0) { part[g * (kGqaDim + 2)] = -INFINITY; part[g * (kGqaDim + 2) + 1] = 0.f; }
        return;
    }
    // q of the group
    const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(a.q_out) + ((size_t)row * a.q_heads + kvh * G) * kGqaDim;
    // K and V blocks: 64 keys x 128 bytes each, rows kv_heads * 128 apart.  All of a thread's loads (four pieces of
    // K, four of V, its q values) are issued before the first is used: one memory round trip after the page number's.
    {
        constexpr int kPieces = kGqaBlock * 8 / kGqaDim;  // 16-byte pieces per thread and block
        const uint8_t* kb = a.k_cache + ((size_t)page * kGqaBlock * a.kv_heads + kvh) * kGqaDim;
        const uint8_t* vbase = a.v_cache + ((size_t)page * kGqaBlock * a.kv_heads + kvh) * kGqaDim;
        uint4 kw[kPieces], vw[kPieces];
        float qv[kGqaMaxGroup];
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
            const int c = tid + i * kGqaDim, key = c >> 3, piece = c & 7;
            kw[i] = *reinterpret_cast<const uint4*>(kb + (size_t)key * a.kv_heads * kGqaDim + piece * 16);
        }
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
            const int c = tid + i * kGqaDim, key = c >> 3, piece = c & 7;
            vw[i] = *reinterpret_cast<const uint4*>(vbase + (size_t)key * a.kv_heads * kGqaDim + piece * 16);
        }
#pragma unroll
        for (int g = 0; g < kGqaMaxGroup; ++g) qv[g] = __bfloat162float(qg[min(g, G - 1) * kGqaDim + tid]);
#pragma unroll
        for (int g = 0; g < kGqaMaxGroup; ++g)
            if (g < G) sm.q[g][tid] = qv[g];
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
            const int c = tid + i * kGqaDim, key = c >> 3, piece = c & 7;
            const uint32_t ws[4] = {kw[i].x, kw[i].y, kw[i].z, kw[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int k = 0; k < 4; ++k) sm.k[key][piece * 16 + j * 4 + k] = e4m3_to_f32((ws[j] >> (8 * k)) & 0xFF);
            *reinterpret_cast<uint4*>(&sm.v[key][piece * 16]) = vw[i];  // V stays bytes
        }
    }
    __syncthreads();
    // scores: thread = (key, half of the group)
    const float qk_scale = a.k_scale * a.sm_scale;
    {
        const int key = tid & 63, half = tid >> 6;
        for (int g = half; g < G; g += 2) {
            float d = 0.f;
#pragma unroll 8
            for (int k = 0; k < kGqaDim; ++k) d += sm.q[g][k] * sm.k[key][k];
            sm.p[g][key] = key < live ? d * qk_scale : -INFINITY;
        }
    }
    __syncthreads();
    // split-local softmax: a warp per head
    for (int g = warp; g < G; g += 4) {
        const float s0 = sm.p[g][lane], s1 = sm.p[g][lane + 32];
        const float m = warp_max(fmaxf(s0, s1));
        const float p0 = lane < live ? expf(s0 - m) : 0.f, p1 = lane + 32 < live ? expf(s1 - m) : 0.f;
        const float l = warp_sum(p0 + p1);
        sm.p[g][lane] = bf16_round(p0);
        sm.p[g][lane + 32] = bf16_round(p1);
        if (lane == 0) { part[g * (kGqaDim + 2)] = m; part[g * (kGqaDim + 2) + 1] = l; }
    }
    __syncthreads();
    // PV: thread = dim
    {
        float acc[kGqaMaxGroup];
#pragma unroll
        for (int g = 0; g < kGqaMaxGroup; ++g) acc[g] = 0.f;
#pragma unroll 8
        for (int key = 0; key < live; ++key) {
            const float v = e4m3_to_f32(sm.v[key][tid]);
#pragma unroll
            for (int g = 0; g < kGqaMaxGroup; ++g)
                if (g < G) acc[g] += sm.p[g][key] * v;
        }
#pragma unroll
        for (int g = 0; g < kGqaMaxGroup; ++g)
            if (g < G) part[g * (kGqaDim + 2) + 2 + tid] = acc[g];
    }
}

// grid (rows * q_heads), 128 threads
__global__ void __launch_bounds__(kGqaDim, 4) gqa_merge_kernel(const mono_gqa_args a) {
    pdl_prologue();
    const int row = blockIdx.x / a.q_heads, h = blockIdx.x - row * a.q_heads, tid = threadIdx.x;
    const int G = a.q_heads / a.kv_heads, kvh = h / G, g = h - kvh * G;
    const float* part = a.scratch + (size_t)(row * a.kv_heads + kvh) * kGqaTopk * G * (kGqaDim + 2) + g * (kGqaDim + 2);
    const size_t stride = (size_t)G * (kGqaDim + 2);
    // every load of the merge is issued before the first is used (a load under a condition waits for the condition:
    // sixteen round trips); a dead split's sum and values are replaced by zeros, which add nothing
    float m[kGqaTopk], l[kGqaTopk], v[kGqaTopk], M = -INFINITY;
#pragma unroll
    for (int j = 0; j < kGqaTopk; ++j) {
        m[j] = part[j * stride];
        l[j] = part[j * stride + 1];
        v[j] = part[j * stride + 2 + tid];
    }
#pragma unroll
    for (int j = 0; j < kGqaTopk; ++j) M = fmaxf(M, m[j]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int j = 0; j < kGqaTopk; ++j) {
        const bool live = m[j] > -INFINITY;
        const float w = live ? expf(m[j] - M) : 0.f;
        num += (live ? v[j] : 0.f) * w;
        den += (live ? l[j] : 0.f) * w;
    }
    const float o = den > 0.f ? num / den * a.v_scale : 0.f;
    reinterpret_cast<__nv_bfloat16*>(a.out)[((size_t)row * a.q_heads + h) * kGqaDim + tid] = __float2bfloat16_rn(o);
}

}  // namespace mono

static int gqa_check(const mono_gqa_args* a, const char* who) {
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->q_heads < 1 || a->kv_heads < 1 || a->q_heads % a->kv_heads ||
        a->q_heads / a->kv_heads > mono::kGqaMaxGroup || !a->positions) {
        mono_set_error("%s: rows 1..16, q_heads a multiple of kv_heads with at most %d q heads per kv head, positions required", who,
                       mono::kGqaMaxGroup);
        return MONO_E_ARG;
    }
    return 0;
}
static int gqa_done(const char* who) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("%s: %s", who, cudaGetErrorString(e));
    return (int)e;
}

extern "C" size_t mono_gqa_scratch_bytes(int rows, int q_heads) {
    return (size_t)rows * q_heads * mono::kGqaTopk * (mono::kGqaDim + 2) * sizeof(float);
}

extern "C" int mono_gqa_front_launch(const mono_gqa_args* a, void* stream) {
    if (int rc = gqa_check(a, "mono_gqa_front_launch")) return rc;
    if (!a->qkv || a->nsum < 1 || !a->g_q || !a->g_k || !a->g_iq || !a->g_ik || !a->cos || !a->sin || !a->k_cache || !a->v_cache ||
        !a->index_cache || !a->q_out || !a->iq_out || !(a->k_scale > 0.f) || !(a->v_scale > 0.f)) {
        mono_set_error("mono_gqa_front_launch: projection sums, norm weights, rope tables, caches with positive scales and outputs required");
        return MONO_E_ARG;
    }
    mono::launch_k(mono::gqa_front_kernel, dim3(a->rows, a->q_heads + 2 * a->kv_heads + 2), mono::kGqaDim, 0, (cudaStream_t)stream, *a);
    return gqa_done("mono_gqa_front_launch");
}

extern "C" int mono_gqa_score_launch(const mono_gqa_args* a, void* stream) {
    if (int rc = gqa_check(a, "mono_gqa_score_launch")) return rc;
    if (!a->iq_out || !a->index_cache || !a->page_table || !a->scores || a->score_ld < 1 || a->score_ld > a->pt_ld || a->n_pages < 1) {
        mono_set_error("mono_gqa_score_launch: index q, an index cache of at least one page, page table and a score buffer of at most pt_ld blocks required");
        return MONO_E_ARG;
    }
    // fp32(fp32(sm_scale) * fp32(log2 e)) as index_score.py:59-62
    const float scale = a->sm_scale * 1.4426950408889634f;
    const int groups = (a->score_ld + mono::kScoreBlocksPerCta - 1) / mono::kScoreBlocksPerCta;
    mono::launch_k(mono::gqa_score_kernel, a->rows * groups, mono::kGqaBlock * mono::kScoreBlocksPerCta, 0, (cudaStream_t)stream, *a, scale);
    return gqa_done("mono_gqa_score_launch");
}

extern "C" int mono_gqa_select_launch(const mono_gqa_args* a, void* stream) {
    if (int rc = gqa_check(a, "mono_gqa_select_launch")) return rc;
    if (!a->scores || !a->page_table || !a->sel_pages || !a->sel_blocks || !a->n_ctx || a->score_ld < 1 ||
        a->score_ld > mono::kSelMaxBlocks || a->init_blocks < 0 || a->local_blocks < 0) {
        mono_set_error("mono_gqa_select_launch: scores of at most %d blocks, page table and selection outputs required", mono::kSelMaxBlocks);
        return MONO_E_ARG;
    }
    const size_t smem = 2 * (size_t)mono::kSelMaxBlocks * sizeof(long long);  // keys + candidates
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        const cudaError_t ae = cudaFuncSetAttribute(mono::gqa_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ae != cudaSuccess) {
            mono_set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(ae));
            return (int)ae;
        }
        mono::attr_done(attr_once);
    }
    mono::launch_k(mono::gqa_select_kernel, a->rows, mono::kSelThreads, smem, (cudaStream_t)stream, *a);
    return gqa_done("mono_gqa_select_launch");
}

extern "C" int mono_gqa_attn_launch(const mono_gqa_args* a, void* stream) {
    if (int rc = gqa_check(a, "mono_gqa_attn_launch")) return rc;
    if (!a->q_out || !a->k_cache || !a->v_cache || !a->sel_pages || !a->n_ctx || !a->scratch || !a->out) {
        mono_set_error("mono_gqa_attn_launch: q, caches, selection, scratch and out required");
        return MONO_E_ARG;
    }
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        const cudaError_t ae = cudaFuncSetAttribute(mono::gqa_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(mono::GqaSplitSmem));
        if (ae != cudaSuccess) {
            mono_set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(ae));
            return (int)ae;
        }
        mono::attr_done(attr_once);
    }
    mono::launch_k(mono::gqa_split_kernel, a->rows * a->kv_heads * mono::kGqaTopk, mono::kGqaDim, sizeof(mono::GqaSplitSmem), (cudaStream_t)stream, *a);
    mono::launch_k(mono::gqa_merge_kernel, a->rows * a->q_heads, mono::kGqaDim, 0, (cudaStream_t)stream, *a);
    return gqa_done("mono_gqa_attn_launch");
}
