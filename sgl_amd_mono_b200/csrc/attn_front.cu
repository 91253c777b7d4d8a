// Attention front stages between the projections: q_a / KV norms, RoPE, the FP8 KV
// cache write, the FP4 index-key write, q post-processing and the W_UK absorb.
//
// Reference counterparts: glm53/gfx950/kernel.py:1978-2003 (q_a RMSNorm), :2005-2101
// (KV RMSNorm, k_pe RoPE, cache row write), :2103-2181 (index key: LayerNorm, RoPE,
// Hadamard, scale + quantise), :2183-2353 (q_b epilogue: RoPE, index q), :2355-2443
// (W_UK absorb); FP4 key format of deepseek_v4/gfx950/kernels/stages/indexer.py:143-151.
#include "mono_common.cuh"
#include "rowdot.cuh"

extern void mono_set_error(const char* fmt, ...);

namespace mono {

constexpr int kMidThreads2 = 256;
MONO_TL_DECLARE(tl_mid)
#ifdef MONO_TIMELINE
#define MID_TL(p) do { if (threadIdx.x == 0) tl_mid[blockIdx.y * 16 + blockIdx.x][p] = globaltimer_ns(); } while (0)
#else
#define MID_TL(p) do { } while (0)
#endif

// hi/lo E4M3 planes of 128 bf16-valued floats held 4 per lane (see MONO_ACT_HILO)
__device__ __forceinline__ void hilo_chunk(const float v[4], int lane, uint8_t* hi, uint8_t* lo, float* scale) {
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = warp_max(amax);
    const int code = code_ceil(fmaxf(amax, 7.888609052210118e-31f) / 448.f);
    const float inv = exp2_code(254 - code);
    uint32_t wh = 0, wl = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float s = v[i] * inv;
        const uint8_t h = f32_to_e4m3(s);
        const uint8_t l = f32_to_e4m3(s - e4m3_to_f32(h));
        wh |= (uint32_t)h << (8 * i);
        wl |= (uint32_t)l << (8 * i);
    }
    reinterpret_cast<uint32_t*>(hi)[lane] = wh;
    reinterpret_cast<uint32_t*>(lo)[lane] = wl;
    if (lane == 0) *scale = exp2_code(code);
}

// In-place orthonormal FWHT over 128 floats in shared memory by 128 threads
// (Sylvester order: butterflies of span 1, 2, 4 ... 64, then * 128^-1/2).
__device__ __forceinline__ void fwht128(float* x, int t /* 0..127 */) {
#pragma unroll
    for (int h = 1; h < 128; h <<= 1) {
        __syncthreads();
        const float a = x[t & ~h], b = x[t | h];
        __syncthreads();
        x[t] = (t & h) ? a - b : a + b;
    }
    __syncthreads();
    x[t] *= 0.08838834764831845f;
    __syncthreads();
}

__global__ void __launch_bounds__(kMidThreads2, 1) mla_mid_kernel(const mono_mla_mid_args a) {
    pdl_launch_dependents();
    MID_TL(0);
    {
        // during the wait for the GEMV before this launch: the norm weights and this row's rotary entries
        // (the step's positions are inputs of the step, not results of that GEMV)
        const int t = threadIdx.x, part_ = blockIdx.y;
        if (part_ == 0) prefetch_span(a.q_a_norm, (size_t)a.q_lora * 2, t, kMidThreads2);
        if (part_ == 1) prefetch_span(a.kv_a_norm, 512 * 2, t, kMidThreads2);
        if (part_ == 2 && a.ik) {
            prefetch_span(a.ik_norm_w, 128 * 4, t, kMidThreads2);
            prefetch_span(a.ik_norm_b, 128 * 4, t, kMidThreads2);
        }
        if (t == 0 && part_ != 0) {
            const int64_t pos_ = a.positions[blockIdx.x];
            prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(a.cos) + pos_ * 32);
            prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(a.sin) + pos_ * 32);
        }
    }
    // grid = (rows, parts): part 0 = q_a, part 1 = latent | rope + cache write, part 2 = index key;
    // the three are independent, so they run on three CTAs instead of one after the other
    const int row = blockIdx.x, part = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // the row's position, slot and rotary entries are inputs of the step: read during the wait as well
    const int64_t pos = a.positions[row];
    const int64_t slot = a.slots ? a.slots[row] : 1;
    float ikraw = 0.f, rc = 0.f, rs = 0.f;
    if (tid < 32 && part != 0) {
        rc = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.cos)[pos * 32 + tid]);
        rs = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.sin)[pos * 32 + tid]);
    }
    // part 0: thread t owns columns 4 t .. 4 t + 3 of each 1024-column stretch of q_a: the four values lane t % 32 holds
    // of chunk (stretch * 8 + warp) when the row is split into hi / lo planes, so the row never goes through shared
    // memory.  Its norm weights are read here, during the wait.
    uint2 qg[2] = {make_uint2(0u, 0u), make_uint2(0u, 0u)};
    if (part == 0) {
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int i = it * kMidThreads2 * 4 + tid * 4;
            qg[it] = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.q_a_norm) + min(i, a.q_lora - 4)));
        }
    }
    MID_TL(1);
    pdl_wait();
    MID_TL(2);
    __shared__ __align__(16) float kv[kKvDim];
    __shared__ float ikv[128];
    __shared__ float red[kMidThreads2 / 32];
    const float* src = a.qkv + (size_t)row * a.ld;
    // everything that does not depend on a reduction is fetched up front
    if (a.ik && part == 2 && tid < 128) {
        for (int s0 = 0; s0 < a.ik_nsum; s0 += 8) {
            float t8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                t8[j] = __ldcg(a.ik + (size_t)min(s0 + j, a.ik_nsum - 1) * a.ik_sum_stride + (size_t)row * a.ik_ld + tid);
#pragma unroll
            for (int j = 0; j < 8; ++j) ikraw += s0 + j < a.ik_nsum ? t8[j] : 0.f;
        }
    }
    // ---- q_a: RMSNorm -> bf16 -> hi/lo planes
    // the whole row (q_a | latent | rope) is summed over the K splits with 16-byte loads
    // issued together, so it costs one memory latency rather than one per element
    float ssq = 0.f, ssq_kv = 0.f;
    if (part == 0) {
        float4 qv[2];
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int i = it * kMidThreads2 * 4 + tid * 4;
            qv[it] = sum_partials4<16>(src + min(i, a.q_lora - 4), a.sum_stride, a.nsum);
            if (i >= a.q_lora) qv[it] = make_float4(0.f, 0.f, 0.f, 0.f);
            ssq += qv[it].x * qv[it].x + qv[it].y * qv[it].y + qv[it].z * qv[it].z + qv[it].w * qv[it].w;
        }
        MID_TL(3);
        const float r = rsqrtf(block_sum<kMidThreads2 / 32>(ssq, red) / (float)a.q_lora + a.eps);
        MID_TL(4);
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int c = it * (kMidThreads2 / 32) + warp;
            if (c < a.q_lora / 128) {  // (the same for a whole warp)
                const float2 glo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qg[it].x));
                const float2 ghi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qg[it].y));
                const float v[4] = {bf16_round(qv[it].x * r * glo.x), bf16_round(qv[it].y * r * glo.y), bf16_round(qv[it].z * r * ghi.x),
                                    bf16_round(qv[it].w * r * ghi.y)};
                uint8_t* hi = a.qa_planes + (size_t)row * a.qa_ld + c * 128;
                hilo_chunk(v, lane, hi, hi + a.qa_plane_stride, a.qa_scale + (size_t)row * a.qa_scale_ld + c);
            }
        }
        MID_TL(5);
        return;
    }
    const int i_lo = a.q_lora, i_hi = part == 1 ? a.q_lora + kKvDim : 0;
    for (int i = i_lo + tid * 4; i < i_hi; i += kMidThreads2 * 4) {
        const float4 v = sum_partials4<16>(src + i, a.sum_stride, a.nsum);
        const float sq = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        *reinterpret_cast<float4*>(kv + (i - a.q_lora)) = v;
        if (i - a.q_lora < 512) ssq_kv += sq;
    }
    MID_TL(3);
    // ---- latent: RMSNorm -> bf16; k_pe: interleaved RoPE -> bf16
    if (part == 1) {
        const float r = rsqrtf(block_sum<kMidThreads2 / 32>(ssq_kv, red) / 512.f + a.eps);
        const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(a.kv_a_norm);
        float rot0 = 0.f, rot1 = 0.f;
        if (tid < 32) {
            const float x0 = kv[512 + 2 * tid], x1 = kv[512 + 2 * tid + 1];
            rot0 = x0 * rc - x1 * rs;
            rot1 = x0 * rs + x1 * rc;
        }
        __syncthreads();
        for (int i = tid; i < 512; i += kMidThreads2) kv[i] = bf16_round(kv[i] * r * __bfloat162float(g[i]));
        if (tid < 32) {
            kv[512 + 2 * tid] = bf16_round(rot0);
            kv[512 + 2 * tid + 1] = bf16_round(rot1);
        }
    }
    if (part == 1) {
    __syncthreads();
    float amax = 0.f;
    for (int i = tid; i < kKvDim; i += kMidThreads2) amax = fmaxf(amax, fabsf(kv[i]));
    amax = block_max<kMidThreads2 / 32>(amax, red);
    if (a.kv_out) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.kv_out) + (size_t)row * kKvDim;
        for (int i = tid; i < kKvDim; i += kMidThreads2) o[i] = __float2bfloat16_rn(kv[i]);
    }
    if (slot >= 0 && slot < a.n_pages * kPage) {
        const int code = code_ceil(fmaxf(amax, 1e-4f) / 448.f);
        const float inv = exp2_code(254 - code);
        uint8_t* page = a.kv_pages + (size_t)(slot / kPage) * kKvPageBytes;
        const int off = (int)(slot % kPage);
        if (tid < kKvDim / 4) {
            uint32_t w = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) w |= (uint32_t)f32_to_e4m3(kv[4 * tid + i] * inv) << (8 * i);
            reinterpret_cast<uint32_t*>(page + (size_t)off * kKvDim)[tid] = w;
        }
        if (tid == 0) reinterpret_cast<float*>(page + kPage * kKvDim)[off] = exp2_code(code);
    }
    MID_TL(5);
    return;
    }
    // ---- index key: LayerNorm -> RoPE (dims 0..63) -> FWHT-128 -> E2M1 + E8M0 per 32
    if (a.ik && part == 2) {
        const float v = ikraw;
        const float mean = block_sum<kMidThreads2 / 32>(tid < 128 ? v : 0.f, red) / 128.f;
        const float dv = tid < 128 ? v - mean : 0.f;
        const float var = block_sum<kMidThreads2 / 32>(dv * dv, red) / 128.f;
        if (tid < 128) ikv[tid] = dv * rsqrtf(var + 1e-6f) * a.ik_norm_w[tid] + a.ik_norm_b[tid];
        __syncthreads();
        float r0 = 0.f, r1 = 0.f;
        if (tid < 32) {
            const float x0 = ikv[2 * tid], x1 = ikv[2 * tid + 1];
            r0 = x0 * rc - x1 * rs;
            r1 = x0 * rs + x1 * rc;
        }
        __syncthreads();
        if (tid < 32) { ikv[2 * tid] = r0; ikv[2 * tid + 1] = r1; }
        // all 256 threads take part in the barriers; threads >= 128 mirror thread - 128
        fwht128(ikv, tid & 127);
        if (tid < 128) {
            const float x = ikv[tid];
            if (a.ik_out) a.ik_out[(size_t)row * 128 + tid] = x;
            float am = fabsf(x);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
            const int code = min(max(code_ceil(fmaxf(am, 6.0f * 1.1754943508222875e-38f) / 6.0f), 1), 254);
            const float q = fminf(fmaxf(x * exp2_code(254 - code), -6.f), 6.f);
            const uint32_t nib = f32_to_e2m1(q);
            const uint32_t other = __shfl_xor_sync(0xffffffffu, nib, 1);
            if (slot >= 0 && slot < a.n_pages * kPage) {
                uint8_t* page = a.idx_pages + (size_t)(slot / kPage) * kIdxPageBytes;
                const int off = (int)(slot % kPage);
                if ((tid & 1) == 0) page[(size_t)off * 64 + (tid >> 1)] = (uint8_t)(nib | (other << 4));
                if ((tid & 31) == 0) page[kPage * 64 + off * 4 + (tid >> 5)] = (uint8_t)code;
            }
        }
    }
    MID_TL(5);
}

// ------------------------------------------------------------------ q_post
// q_post_kernel, 8 * heads blocks: one (head, 64 latent columns) each, all rows: q_nope -> bf16,
// W_UK absorb; the first block of a head also writes the rotated q_pe.
// q_post_index_kernel, rows * index_heads blocks: one index query each.
constexpr int kQPostThreads = 128;

__global__ void __launch_bounds__(kQPostThreads) q_post_kernel(const mono_q_post_args a) {
    pdl_launch_dependents();
    __shared__ __align__(16) float qn[kMaxRows][128];
    const int tid = threadIdx.x;
    const __nv_bfloat16* cosb = reinterpret_cast<const __nv_bfloat16*>(a.cos);
    const __nv_bfloat16* sinb = reinterpret_cast<const __nv_bfloat16*>(a.sin);
    if ((int)blockIdx.x < a.heads * 8) {
        // one block per (head, 64-column slab of the latent): 8 x heads blocks keep every SM busy
        const int h = blockIdx.x >> 3, cq0 = blockIdx.x & 7;
        __nv_bfloat16* qf = reinterpret_cast<__nv_bfloat16*>(a.q_full);
        // During the wait for the GEMV before this launch: this block's 128 x 64-byte slab of W_UK (all 512
        // sixteen-byte loads issued before any is used, 4 per thread), stored transposed ([column][d], so that
        // a thread reads four d of its column in one word), and, in the block that rotates q_pe, every row's
        // rotary entries (positions and tables are inputs of the step).
        __shared__ __align__(16) uint8_t wt[64][128 + 4];
        __shared__ float rot[2][kMaxRows][32];
        {
            uint4 wv4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = tid + i * kQPostThreads;  // 0..511: row d = idx / 4, 16-byte piece idx % 4
                wv4[i] = __ldg(reinterpret_cast<const uint4*>(a.kv_b + ((size_t)h * 256 + (idx >> 2)) * 512 + cq0 * 64) + (idx & 3));
            }
            if (cq0 == 0 && tid < 32) {
                int64_t pos[kMaxRows];
#pragma unroll
                for (int r = 0; r < kMaxRows; ++r) pos[r] = a.positions[min(r, a.rows - 1)];
#pragma unroll
                for (int r = 0; r < kMaxRows; ++r) {
                    rot[0][r][tid] = __bfloat162float(cosb[pos[r] * 32 + tid]);
                    rot[1][r][tid] = __bfloat162float(sinb[pos[r] * 32 + tid]);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = tid + i * kQPostThreads;
                const uint32_t w[4] = {wv4[i].x, wv4[i].y, wv4[i].z, wv4[i].w};
#pragma unroll
                for (int j = 0; j < 16; ++j) wt[(idx & 3) * 16 + j][idx >> 2] = (uint8_t)(w[j >> 2] >> (8 * (j & 3)));
            }
        }
        const float wsc = a.kv_b_scale[(size_t)(h * 2) * 4 + (cq0 * 64) / 128];
        pdl_wait();
        // the rows' q_nope: one batch of loads per K split, all rows in flight together
        {
            float v[kMaxRows];
#pragma unroll
            for (int r = 0; r < kMaxRows; ++r) v[r] = 0.f;
            for (int s = 0; s < a.nsum; ++s) {
                float t[kMaxRows];
#pragma unroll
                for (int r = 0; r < kMaxRows; ++r)
                    t[r] = __ldcg(a.qb + (size_t)s * a.sum_stride + (size_t)min(r, a.rows - 1) * a.ld + h * 192 + tid);
#pragma unroll
                for (int r = 0; r < kMaxRows; ++r) v[r] += t[r];  // rows past the last repeat the last row: not stored below
            }
#pragma unroll
            for (int r = 0; r < kMaxRows; ++r) qn[r][tid] = r < a.rows ? bf16_round(v[r]) : 0.f;
        }
        if (cq0 == 0 && tid < 32) {  // q_pe: interleaved rotation of the head's last 64 values
            float2 xp[kMaxRows];
#pragma unroll
            for (int r = 0; r < kMaxRows; ++r) xp[r] = make_float2(0.f, 0.f);
            for (int s = 0; s < a.nsum; ++s) {
                float2 t2[kMaxRows];
#pragma unroll
                for (int r = 0; r < kMaxRows; ++r)
                    t2[r] = __ldcg(reinterpret_cast<const float2*>(a.qb + (size_t)s * a.sum_stride + (size_t)min(r, a.rows - 1) * a.ld + h * 192 + 128) + tid);
#pragma unroll
                for (int r = 0; r < kMaxRows; ++r) { xp[r].x += t2[r].x; xp[r].y += t2[r].y; }
            }
#pragma unroll
            for (int r = 0; r < kMaxRows; ++r) {
                if (r < a.rows) {
                    const float c = rot[0][r][tid], sn = rot[1][r][tid];
                    __nv_bfloat16* o = qf + ((size_t)r * a.heads + h) * kKvDim + 512;
                    o[2 * tid] = __float2bfloat16_rn(xp[r].x * c - xp[r].y * sn);
                    o[2 * tid + 1] = __float2bfloat16_rn(xp[r].x * sn + xp[r].y * c);
                }
            }
        }
        __syncthreads();
        // q_lat[c] = sum_d W_UK[d][c] * q_nope[d], d ascending.  thread = (column c = tid % 64, row half = tid / 64):
        // rows half, half + 2, ...; four d per step: one word of weights, one float4 of each row's q_nope
        const int c = tid & 63, half = tid >> 6;
        const int nr = (a.rows + 1 - half) >> 1;  // rows of this half that exist
        float acc[kMaxRows / 2];
#pragma unroll
        for (int r = 0; r < kMaxRows / 2; ++r) acc[r] = 0.f;
#pragma unroll 4
        for (int d0 = 0; d0 < 128; d0 += 4) {
            const uint32_t w4 = *reinterpret_cast<const uint32_t*>(&wt[c][d0]);
            const float w0 = e4m3_to_f32((uint8_t)w4), w1 = e4m3_to_f32((uint8_t)(w4 >> 8)), w2 = e4m3_to_f32((uint8_t)(w4 >> 16)),
                        w3 = e4m3_to_f32((uint8_t)(w4 >> 24));
#pragma unroll
            for (int r = 0; r < kMaxRows / 2; ++r) {
                if (r < nr) {
                    const float4 q4 = *reinterpret_cast<const float4*>(&qn[2 * r + half][d0]);
                    acc[r] = fmaf(q4.x, w0, acc[r]);
                    acc[r] = fmaf(q4.y, w1, acc[r]);
                    acc[r] = fmaf(q4.z, w2, acc[r]);
                    acc[r] = fmaf(q4.w, w3, acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < kMaxRows / 2; ++r) {
            const int row = 2 * r + half;
            if (row < a.rows) qf[((size_t)row * a.heads + h) * kKvDim + cq0 * 64 + c] = __float2bfloat16_rn(acc[r] * wsc);
        }
    }
}

// One index query (row r, index head ih) by the first 128 threads of a block; every thread of the block calls this
// (the Hadamard butterflies hold block-wide barriers; threads past 127 mirror thread - 128).
__device__ __forceinline__ void index_query_body(const mono_q_post_args& a, int idx, int tid, float* iq) {
    const __nv_bfloat16* cosb = reinterpret_cast<const __nv_bfloat16*>(a.cos);
    const __nv_bfloat16* sinb = reinterpret_cast<const __nv_bfloat16*>(a.sin);
    const int r = idx / a.index_heads, ih = idx - r * a.index_heads, t = tid & 127;
    float c = 0.f, sn = 0.f;
    if (tid < 32) {  // inputs of the step: read during the wait
        const int64_t pos = a.positions[r];
        c = __bfloat162float(cosb[pos * 32 + tid]);
        sn = __bfloat162float(sinb[pos * 32 + tid]);
    }
    pdl_wait();
    const float* src = a.iq + (size_t)r * a.iq_ld + ih * 128;
    float v = 0.f;
    for (int s0 = 0; s0 < a.iq_nsum; s0 += 4) {
        float t4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) t4[j] = __ldcg(src + (size_t)min(s0 + j, a.iq_nsum - 1) * a.iq_sum_stride + t);
#pragma unroll
        for (int j = 0; j < 4; ++j) v += s0 + j < a.iq_nsum ? t4[j] : 0.f;
    }
    if (tid < 128) iq[t] = v;
    __syncthreads();
    float r0 = 0.f, r1 = 0.f;
    if (tid < 32) {
        const float x0 = iq[2 * tid], x1 = iq[2 * tid + 1];
        r0 = x0 * c - x1 * sn;
        r1 = x0 * sn + x1 * c;
    }
    __syncthreads();
    if (tid < 32) { iq[2 * tid] = r0; iq[2 * tid + 1] = r1; }
    fwht128(iq, t);
    if (tid < 128) reinterpret_cast<__nv_bfloat16*>(a.idx_q)[((size_t)r * a.index_heads + ih) * 128 + t] = __float2bfloat16_rn(iq[t]);
}

// The index queries alone: a kernel of its own, so that its small blocks (few registers, 1 KB of shared memory) find
// room on SMs that the head blocks of q_post_kernel already fill while they wait for the same projection.
__global__ void __launch_bounds__(kQPostThreads) q_post_index_kernel(const mono_q_post_args a) {
    pdl_launch_dependents();
    __shared__ float iq[128];
    index_query_body(a, blockIdx.x, threadIdx.x, iq);
}

// The index queries and the index head weights (x @ weights_proj) in one launch: the two inputs of the score launch
// that are not there yet when the q_b projection ends.  Blocks [0, d.n): one head-weight column each (the body of
// rowdot_kernel; they need the normed input only and are done before the projection is); the rest: one index query
// each.  One launch on the step's longer branch instead of two.
__global__ void __launch_bounds__(kRowdotThreads, 2) index_prep_kernel(const mono_q_post_args a, const mono_rowdot_args d) {
    pdl_launch_dependents();
    __shared__ float red[1][kRowdotThreads / 32][kMaxRows];
    __shared__ float iq[128];
    if ((int)blockIdx.x < d.n) rowdot_col<1, false>(d, blockIdx.x, threadIdx.x, red);
    else index_query_body(a, blockIdx.x - d.n, threadIdx.x, iq);
}

}  // namespace mono

#ifdef MONO_TIMELINE
extern "C" int mono_timeline_read_mla_mid(unsigned long long* out, int* ctas, int* points) {
    *ctas = MONO_TL_CTAS;
    *points = MONO_TL_POINTS;
    return (int)cudaMemcpyFromSymbol(out, mono::tl_mid, sizeof(unsigned long long) * MONO_TL_CTAS * MONO_TL_POINTS);
}
#endif

extern "C" int mono_mla_mid_launch(const mono_mla_mid_args* a, void* stream) {
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->q_lora < 128 || a->q_lora > 2048 || (a->q_lora & 127) || !a->qkv ||
        !a->q_a_norm || !a->kv_a_norm || !a->cos || !a->sin || !a->positions || !a->qa_planes || !a->qa_scale || !a->kv_pages) {
        mono_set_error("mono_mla_mid_launch: rows 1..16, q_lora a multiple of 128 up to 2048 and all pointers required");
        return MONO_E_ARG;
    }
    if (a->ik && (!a->ik_norm_w || !a->ik_norm_b || !a->idx_pages)) {
        mono_set_error("mono_mla_mid_launch: an index key needs its norm weights and the index pages");
        return MONO_E_ARG;
    }
    mono::launch_k(mono::mla_mid_kernel, dim3(a->rows, a->ik ? 3 : 2), mono::kMidThreads2, 0, (cudaStream_t)stream, *a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_mla_mid_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

extern "C" int mono_index_prep_launch(const mono_q_post_args* a, const mono_rowdot_args* d, void* stream) {
    if (!a || !d || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->index_heads < 1 || !a->cos || !a->sin || !a->positions || !a->iq ||
        !a->idx_q || d->rows != a->rows || d->n < 1 || d->k < 128 || (d->k & 127) || !d->w || !d->x_bf16 || !d->out) {
        mono_set_error("mono_index_prep_launch: rows 1..16, index heads with their partial sums and output, and a row-dot over "
                       "the same rows (k a multiple of 128) required");
        return MONO_E_ARG;
    }
    mono::launch_k(mono::index_prep_kernel, d->n + a->rows * a->index_heads, mono::kRowdotThreads, 0, (cudaStream_t)stream, *a, *d);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_index_prep_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

extern "C" int mono_q_post_launch(const mono_q_post_args* a, void* stream) {
    // heads == 0 runs the index queries alone, index_heads == 0 the head part alone: the two halves are
    // independent and may run on different streams
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->heads < 0 || a->index_heads < 0 || (a->heads == 0 && a->index_heads == 0) ||
        !a->cos || !a->sin || !a->positions || (a->heads > 0 && (!a->qb || !a->kv_b || !a->kv_b_scale || !a->q_full)) ||
        (a->index_heads > 0 && (!a->iq || !a->idx_q))) {
        mono_set_error("mono_q_post_launch: rows 1..16, heads and / or index_heads > 0 with their pointers required");
        return MONO_E_ARG;
    }
    // the index queries first: the launch after them (the scores) is the longer path of the two
    if (a->index_heads > 0) mono::launch_k(mono::q_post_index_kernel, a->rows * a->index_heads, mono::kQPostThreads, 0, (cudaStream_t)stream, *a);
    if (a->heads > 0) mono::launch_k(mono::q_post_kernel, a->heads * 8, mono::kQPostThreads, 0, (cudaStream_t)stream, *a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_q_post_launch: %s", cudaGetErrorString(e));
    return (int)e;
}
