// Attention front stages between the projections: q_a / KV norms, RoPE, the FP8 KV
// cache write, the FP4 index-key write, q post-processing and the W_UK absorb.
//
// Reference counterparts: glm53/gfx950/kernel.py:1978-2003 (q_a RMSNorm), :2005-2101
// (KV RMSNorm, k_pe RoPE, cache row write), :2103-2181 (index key: LayerNorm, RoPE,
// Hadamard, scale + quantise), :2183-2353 (q_b epilogue: RoPE, index q), :2355-2443
// (W_UK absorb); FP4 key format of deepseek_v4/gfx950/kernels/stages/indexer.py:143-151.
#include "mono_common.cuh"

extern void mono_set_error(const char* fmt, ...);

namespace mono {

constexpr int kMidThreads2 = 256;

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

__global__ void __launch_bounds__(kMidThreads2) mla_mid_kernel(const mono_mla_mid_args a) {
    pdl_launch_dependents();
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
    pdl_wait();
    __shared__ __align__(16) float xq[2048 + 64];
    __shared__ __align__(16) float kv[kKvDim];
    __shared__ float ikv[128];
    __shared__ float red[kMidThreads2 / 32];
    // grid = (rows, parts): part 0 = q_a, part 1 = latent | rope + cache write, part 2 = index key;
    // the three are independent, so they run on three CTAs instead of one after the other
    const int row = blockIdx.x, part = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t pos = a.positions[row];
    const int64_t slot = a.slots ? a.slots[row] : 1;
    const float* src = a.qkv + (size_t)row * a.ld;
    // everything that does not depend on a reduction is fetched up front
    float ikraw = 0.f, rc = 0.f, rs = 0.f;
    if (a.ik && part == 2 && tid < 128) {
#pragma unroll 4
        for (int s = 0; s < a.ik_nsum; ++s) ikraw += a.ik[(size_t)s * a.ik_sum_stride + (size_t)row * a.ik_ld + tid];
    }
    if (tid < 32) {
        rc = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.cos)[pos * 32 + tid]);
        rs = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.sin)[pos * 32 + tid]);
    }
    // ---- q_a: RMSNorm -> bf16 -> hi/lo planes
    // the whole row (q_a | latent | rope) is summed over the K splits with 16-byte loads
    // issued together, so it costs one memory latency rather than one per element
    float ssq = 0.f, ssq_kv = 0.f;
    const int i_lo = part == 0 ? 0 : a.q_lora, i_hi = part == 0 ? a.q_lora : (part == 1 ? a.q_lora + kKvDim : 0);
    for (int i = i_lo + tid * 4; i < i_hi; i += kMidThreads2 * 4) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int s = 0; s < a.nsum; ++s) {
            const float4 p = *reinterpret_cast<const float4*>(src + (size_t)s * a.sum_stride + i);
            v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
        }
        const float sq = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        if (i < a.q_lora) {
            *reinterpret_cast<float4*>(xq + i) = v;
            ssq += sq;
        } else {
            *reinterpret_cast<float4*>(kv + (i - a.q_lora)) = v;
            if (i - a.q_lora < 512) ssq_kv += sq;
        }
    }
    if (part == 0) {
        const float r = rsqrtf(block_sum<kMidThreads2 / 32>(ssq, red) / (float)a.q_lora + a.eps);
        const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(a.q_a_norm);
        for (int i = tid; i < a.q_lora; i += kMidThreads2) xq[i] = bf16_round(xq[i] * r * __bfloat162float(g[i]));
        __syncthreads();
        for (int c = warp; c < a.q_lora / 128; c += kMidThreads2 / 32) {
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = xq[c * 128 + 4 * lane + i];
            uint8_t* hi = a.qa_planes + (size_t)row * a.qa_ld + c * 128;
            hilo_chunk(v, lane, hi, hi + a.qa_plane_stride, a.qa_scale + (size_t)row * a.qa_scale_ld + c);
        }
        return;
    }
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
}

// ------------------------------------------------------------------ q_post
// blocks [0, 8 * heads): one (head, 64 latent columns) each, all rows: q_nope -> bf16,
// W_UK absorb; the first block of a head also writes the rotated q_pe.
// blocks [8 * heads, 8 * heads + rows * index_heads): one index query each.
constexpr int kQPostThreads = 128;

__global__ void __launch_bounds__(kQPostThreads) q_post_kernel(const mono_q_post_args a) {
    pdl_launch_dependents();
    if ((int)blockIdx.x < a.heads * 8) {
        // during the wait for the GEMV before this launch: this block's 128 x 64-byte slab of W_UK
        const int h_ = blockIdx.x >> 3, cq_ = blockIdx.x & 7;
        prefetch_l2(a.kv_b + ((size_t)h_ * 256 + threadIdx.x) * 512 + cq_ * 64);
    }
    pdl_wait();
    __shared__ float qn[kMaxRows][128];
    __shared__ float iq[128];
    const int tid = threadIdx.x;
    const __nv_bfloat16* cosb = reinterpret_cast<const __nv_bfloat16*>(a.cos);
    const __nv_bfloat16* sinb = reinterpret_cast<const __nv_bfloat16*>(a.sin);
    if ((int)blockIdx.x < a.heads * 8) {
        // one block per (head, 64-column slab of the latent): 8 x heads blocks keep every SM busy
        const int h = blockIdx.x >> 3, cq0 = blockIdx.x & 7;
        __nv_bfloat16* qf = reinterpret_cast<__nv_bfloat16*>(a.q_full);
        for (int r = a.rows; r < kMaxRows; ++r) qn[r][tid] = 0.f;
#pragma unroll 4
        for (int r = 0; r < a.rows; ++r) {
            const float* src = a.qb + (size_t)r * a.ld + h * 192;
            float v = 0.f;
#pragma unroll 4
            for (int s = 0; s < a.nsum; ++s) v += src[(size_t)s * a.sum_stride + tid];
            qn[r][tid] = bf16_round(v);
            if (cq0 == 0 && tid < 32) {
                float x0 = 0.f, x1 = 0.f;
                for (int s = 0; s < a.nsum; ++s) {
                    x0 += src[(size_t)s * a.sum_stride + 128 + 2 * tid];
                    x1 += src[(size_t)s * a.sum_stride + 128 + 2 * tid + 1];
                }
                const int64_t pos = a.positions[r];
                const float c = __bfloat162float(cosb[pos * 32 + tid]), sn = __bfloat162float(sinb[pos * 32 + tid]);
                __nv_bfloat16* o = qf + ((size_t)r * a.heads + h) * kKvDim + 512;
                o[2 * tid] = __float2bfloat16_rn(x0 * c - x1 * sn);
                o[2 * tid + 1] = __float2bfloat16_rn(x0 * sn + x1 * c);
            }
        }
        // q_lat[c] = sum_d W_UK[d][c] * q_nope[d].  All 512 sixteen-byte loads of a
        // 128 x 64-column slab are issued before any is used (4 per thread), so the
        // 64 KB of a head arrive in four latency periods instead of 128.
        __shared__ __align__(16) uint8_t wt[128][64 + 16];
        for (int cq = cq0; cq < cq0 + 1; ++cq) {
            __syncthreads();
            uint4 v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = tid + i * kQPostThreads;  // 0..511: row d = idx / 4, 16-byte piece idx % 4
                v[i] = __ldg(reinterpret_cast<const uint4*>(a.kv_b + ((size_t)h * 256 + (idx >> 2)) * 512 + cq * 64) + (idx & 3));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = tid + i * kQPostThreads;
                *reinterpret_cast<uint4*>(&wt[idx >> 2][(idx & 3) * 16]) = v[i];
            }
            __syncthreads();
            // thread = (column c = tid % 64, row half = tid / 64): rows r = half, half + 2, ...
            const int c = tid & 63, half = tid >> 6;
            float acc[kMaxRows / 2];
#pragma unroll
            for (int r = 0; r < kMaxRows / 2; ++r) acc[r] = 0.f;
#pragma unroll 8
            for (int d = 0; d < 128; ++d) {
                const float w = e4m3_to_f32(wt[d][c]);
#pragma unroll
                for (int r = 0; r < kMaxRows / 2; ++r) acc[r] += qn[2 * r + half][d] * w;
            }
            const float sc = a.kv_b_scale[(size_t)(h * 2) * 4 + (cq * 64) / 128];
#pragma unroll
            for (int r = 0; r < kMaxRows / 2; ++r) {
                const int row = 2 * r + half;
                if (row < a.rows) qf[((size_t)row * a.heads + h) * kKvDim + cq * 64 + c] = __float2bfloat16_rn(acc[r] * sc);
            }
        }
    } else {
        const int idx = blockIdx.x - a.heads * 8;
        const int r = idx / a.index_heads, ih = idx - r * a.index_heads;
        const float* src = a.iq + (size_t)r * a.iq_ld + ih * 128;
        float v = 0.f;
        for (int s = 0; s < a.iq_nsum; ++s) v += src[(size_t)s * a.iq_sum_stride + tid];
        iq[tid] = v;
        __syncthreads();
        float r0 = 0.f, r1 = 0.f;
        if (tid < 32) {
            const int64_t pos = a.positions[r];
            const float c = __bfloat162float(cosb[pos * 32 + tid]), sn = __bfloat162float(sinb[pos * 32 + tid]);
            const float x0 = iq[2 * tid], x1 = iq[2 * tid + 1];
            r0 = x0 * c - x1 * sn;
            r1 = x0 * sn + x1 * c;
        }
        __syncthreads();
        if (tid < 32) { iq[2 * tid] = r0; iq[2 * tid + 1] = r1; }
        fwht128(iq, tid);
        reinterpret_cast<__nv_bfloat16*>(a.idx_q)[((size_t)r * a.index_heads + ih) * 128 + tid] = __float2bfloat16_rn(iq[tid]);
    }
}

}  // namespace mono

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

extern "C" int mono_q_post_launch(const mono_q_post_args* a, void* stream) {
    // heads == 0 runs the index queries alone, index_heads == 0 the head part alone: the two halves are
    // independent and may run on different streams
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->heads < 0 || a->index_heads < 0 || (a->heads == 0 && a->index_heads == 0) ||
        !a->cos || !a->sin || !a->positions || (a->heads > 0 && (!a->qb || !a->kv_b || !a->kv_b_scale || !a->q_full)) ||
        (a->index_heads > 0 && (!a->iq || !a->idx_q))) {
        mono_set_error("mono_q_post_launch: rows 1..16, heads and / or index_heads > 0 with their pointers required");
        return MONO_E_ARG;
    }
    const int blocks = a->heads * 8 + (a->index_heads > 0 ? a->rows * a->index_heads : 0);
    mono::launch_k(mono::q_post_kernel, blocks, mono::kQPostThreads, 0, (cudaStream_t)stream, *a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_q_post_launch: %s", cudaGetErrorString(e));
    return (int)e;
}
