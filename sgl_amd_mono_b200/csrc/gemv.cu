// Weight-streaming GEMV for 1..16 activation rows: the hot loop of every projection
// and of the shared + routed experts.
//
// Reference counterpart: the MFMA GEMV units of glm53/gfx950/kernel.py:1061-1172
// (mma_units), used by q_a|kv_a (:1781), q_b (:2183), W_UV (:3975), o_proj (:4125),
// expert up/gate (:4352-4999) and down (:5001-5187); MXFP4 experts as
// glm53_flash/gfx950/kernel.py:4025-4392.  Same arithmetic contract: weights map to
// the MMA M dimension, the step's rows to N, f32 accumulation per 128-k chunk times
// the 128x128 block scale (kernel.py:35-42), partial sums handed on in f32.
//
// sm_100a design: a persistent grid (one CTA per SM) walks a static task list.  One
// producer warp streams 128-row x 128-byte weight boxes with TMA (128-byte swizzle,
// read in place from SGLang's row-major tensors) into an mbarrier ring and stages each
// segment's activation planes with bulk copies; eight consumer warps issue FP8 / BF16
// tensor-core MMAs straight from the swizzled tiles.  The K order inside an MMA is
// permuted (each thread owns 32 contiguous bytes of a row) so that both operands are
// read with conflict-free 16-byte shared loads; a dot product does not care.
#include "mono_common.cuh"

namespace mono {

constexpr int kTileBytes = 128 * 128;
constexpr int kConsumerWarps = 8;
constexpr int kGemvThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxAStages = 8;
constexpr int kMaxBSlots = 8;

struct GemvParams {
    mono_gemv_args a;
    int a_stages, n_bslots, bslot_bytes;
    int b_pitch;       // bytes per activation row in a slot
    int bb;            // activation bytes per weight tile (128, or 256 for MXFP4)
    int scale_off;     // offset of the scale area inside a slot
    int scale_pitch;   // bytes per scale row
};

struct Seg {
    int c2, row0, t0, nt;
    const uint8_t* act;
    const void* asc;
    const void* wsc;  // FP8: float* for this row block; MXFP4: uint8* row 0 of the block
    const float* coef;
};

__device__ __forceinline__ int job_nrb(const mono_gemv_job& j) { return (j.n_rows + 127) >> 7; }

template <int WK>
__device__ __forceinline__ Seg make_seg(const mono_gemv_job& j, int rb, int ks, int u, int U, int bb) {
    Seg s;
    int mat = 0, rbm = rb;
    if (j.mode == MONO_JOB_DENSE) {
        if (j.rb_per_mat > 0) { mat = rb / j.rb_per_mat; rbm = rb - mat * j.rb_per_mat; }
        s.t0 = ks * j.split_tiles;
        s.nt = min(j.split_tiles, j.k_tiles - s.t0);
        s.act = j.act + (size_t)mat * j.act_seg_stride;
        s.coef = nullptr;
    } else if (j.mode == MONO_JOB_EXPERT_UP) {
        mat = j.expert_list[u];
        s.t0 = ks * j.split_tiles;
        s.nt = min(j.split_tiles, j.k_tiles - s.t0);
        s.act = j.act;
        s.coef = nullptr;
    } else {
        mat = j.expert_list[u];
        s.t0 = 0;
        s.nt = j.k_tiles;
        s.act = j.act + (size_t)u * j.act_seg_stride;
        s.coef = j.coef ? j.coef + (size_t)u * kMaxRows : nullptr;
    }
    (void)U;
    s.c2 = mat;
    s.row0 = j.row_off + rbm * 128;
    const int aseg = (j.mode == MONO_JOB_EXPERT_DOWN) ? u : ((j.mode == MONO_JOB_DENSE) ? mat : 0);
    s.act += (size_t)s.t0 * bb;
    if (WK == MONO_W_FP8) {
        s.asc = j.ascale_f32 + (size_t)aseg * j.ascale_seg_stride + s.t0;
        s.wsc = j.wscale_f32 + (size_t)mat * j.wscale_mat_stride + (size_t)(s.row0 >> 7) * j.wscale_ld + s.t0;
    } else if (WK == MONO_W_MXFP4) {
        s.asc = j.ascale_e8 + (size_t)aseg * j.ascale_seg_stride + (size_t)s.t0 * 8;
        s.wsc = j.wscale_e8 + (size_t)mat * j.wscale_mat_stride + (size_t)s.row0 * j.wscale_ld + (size_t)s.t0 * 8;
    } else {
        s.asc = nullptr;
        s.wsc = nullptr;
    }
    return s;
}

// e2m1 nibbles -> E4M3 bytes of value * 2^-6: the 3 magnitude bits land in E4M3's
// low exponent / top mantissa bits (also right for the E2M1 subnormal 0.5).
__device__ __forceinline__ uint32_t fp4_lo_to_e4m3(uint32_t w) {
    return ((w << 2) & 0x1C1C1C1Cu) | ((w << 4) & 0x80808080u);
}
__device__ __forceinline__ uint32_t fp4_hi_to_e4m3(uint32_t w) {
    return ((w >> 2) & 0x1C1C1C1Cu) | (w & 0x80808080u);
}

template <int WK, int NT>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_ring = smem;
    uint8_t* b_ring = smem + p.a_stages * kTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(b_ring + (size_t)p.n_bslots * p.bslot_bytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + kMaxAStages;
    uint64_t* bfull = bars + 2 * kMaxAStages;
    uint64_t* bempty = bars + 2 * kMaxAStages + kMaxBSlots;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int NPAD = NT * 8;

    if (tid == 0) {
        abort_flag = guard_failed(p.a.guard) ? 1 : 0;
        for (int i = 0; i < kMaxAStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], kConsumerWarps); }
        for (int i = 0; i < kMaxBSlots; ++i) { mbar_init(&bfull[i], 1); mbar_init(&bempty[i], kConsumerWarps); }
        mbar_fence_init();
    }
    __syncthreads();

    // Let the next launch start its prologue, and request the first weight tiles of this
    // CTA's first task before waiting for the previous launch: weights do not depend on
    // anything upstream, so they stream while the predecessor is still finishing.
    pdl_launch_dependents();
    int pre = 0;
    if (warp == kConsumerWarps) {
        const mono_gemv_job& j0 = p.a.job[0];
        if (lane == 0 && j0.mode == MONO_JOB_DENSE) {
            const int nrb0 = j0.rb_per_mat > 0 ? j0.n_mats * j0.rb_per_mat : job_nrb(j0);
            if ((int)blockIdx.x < nrb0 * j0.nsplit) {
                const Seg s0 = make_seg<WK>(j0, blockIdx.x % nrb0, blockIdx.x / nrb0, 0, 0, p.bb);
                pre = min(s0.nt, p.a_stages);
                for (int t = 0; t < pre; ++t) {
                    mbar_expect_tx(&full[t], kTileBytes);
                    tma_load_3d(a_ring + (size_t)t * kTileBytes, reinterpret_cast<const CUtensorMap*>(&j0.tmap),
                                (s0.t0 + t) * 128, s0.row0, s0.c2, &full[t]);
                }
            }
        }
        pre = __shfl_sync(0xffffffffu, pre, 0);
    }
    pdl_wait();

    // task counts (identical in every thread)
    int cnt[MONO_GEMV_MAX_JOBS];
    int nexp[MONO_GEMV_MAX_JOBS];
    int total = 0;
#pragma unroll
    for (int j = 0; j < MONO_GEMV_MAX_JOBS; ++j) {
        cnt[j] = 0;
        nexp[j] = 0;
        if (j < p.a.njobs) {
            const mono_gemv_job& jb = p.a.job[j];
            int nrb = job_nrb(jb);
            if (jb.mode == MONO_JOB_DENSE) {
                cnt[j] = (jb.rb_per_mat > 0 ? jb.n_mats * jb.rb_per_mat : nrb) * jb.nsplit;
            } else {
                int U = min(*jb.n_expert, jb.max_expert);
                nexp[j] = U;
                // down tasks always run: a group without experts writes zeros to its slice
                cnt[j] = (jb.mode == MONO_JOB_EXPERT_UP) ? U * nrb * jb.nsplit : nrb * jb.nsplit;
            }
        }
        total += cnt[j];
    }

    volatile int* abortp = &abort_flag;
    const uint64_t wait_ns = p.a.wait_ns ? p.a.wait_ns : kWaitLimitNs;

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            for (int j = 0; j < p.a.njobs; ++j) prefetch_tmap(reinterpret_cast<const CUtensorMap*>(&p.a.job[j].tmap));
        }
        int astage = 0, bslot = 0;
        uint32_t aphase = 0, bphase = 0;
        for (int task = blockIdx.x; task < total && !*abortp; task += gridDim.x) {
            int j = 0, local = task;
            while (local >= cnt[j]) { local -= cnt[j]; ++j; }
            const mono_gemv_job& jb = p.a.job[j];
            const int nrb = (jb.mode == MONO_JOB_DENSE && jb.rb_per_mat > 0) ? jb.n_mats * jb.rb_per_mat : job_nrb(jb);
            int u = 0, rb, ks, nseg = 1;
            if (jb.mode == MONO_JOB_EXPERT_UP) {
                u = local / (nrb * jb.nsplit);
                local -= u * nrb * jb.nsplit;
            }
            rb = local % nrb;
            ks = local / nrb;
            if (jb.mode == MONO_JOB_EXPERT_DOWN) nseg = (nexp[j] > ks) ? (nexp[j] - ks + jb.nsplit - 1) / jb.nsplit : 0;
            for (int sgi = 0; sgi < nseg; ++sgi) {
                if (jb.mode == MONO_JOB_EXPERT_DOWN) u = ks + sgi * jb.nsplit;
                Seg s = make_seg<WK>(jb, rb, ks, u, nexp[j], p.bb);
                // activation planes + scales of this segment
                int ok = 1;
                if (lane == 0) ok = mbar_wait(&bempty[bslot], bphase ^ 1, abortp, wait_ns) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                uint8_t* slot = b_ring + (size_t)bslot * p.bslot_bytes;
                const uint32_t row_bytes = (uint32_t)s.nt * p.bb;
                uint32_t sc_bytes = 0;
                if (WK == MONO_W_FP8) sc_bytes = (uint32_t)((s.nt + 3) & ~3) * 4;
                if (WK == MONO_W_MXFP4) sc_bytes = (uint32_t)((s.nt * 8 + 15) & ~15);
                if (lane == 0) mbar_expect_tx(&bfull[bslot], (row_bytes * jb.planes + sc_bytes) * NPAD);
                __syncwarp();
                for (int r = lane; r < NPAD * jb.planes; r += 32) {
                    int pl = r / NPAD, row = r - pl * NPAD;
                    bulk_load(slot + (size_t)r * p.b_pitch, s.act + (size_t)pl * jb.act_plane_stride + (size_t)row * jb.act_ld,
                              row_bytes, &bfull[bslot]);
                }
                if (WK == MONO_W_FP8) {
                    for (int r = lane; r < NPAD; r += 32)
                        bulk_load(slot + p.scale_off + (size_t)r * p.scale_pitch,
                                  reinterpret_cast<const float*>(s.asc) + (size_t)r * jb.ascale_ld, sc_bytes, &bfull[bslot]);
                } else if (WK == MONO_W_MXFP4) {
                    for (int r = lane; r < NPAD; r += 32)
                        bulk_load(slot + p.scale_off + (size_t)r * p.scale_pitch,
                                  reinterpret_cast<const uint8_t*>(s.asc) + (size_t)r * jb.ascale_ld, sc_bytes, &bfull[bslot]);
                }
                if (++bslot == p.n_bslots) { bslot = 0; bphase ^= 1; }
                // weight tiles
                if (lane == 0) {
                    for (int t = 0; t < s.nt; ++t) {
                        if (pre > 0) {  // requested before the dependency wait (first task of this CTA)
                            --pre;
                            if (++astage == p.a_stages) { astage = 0; aphase ^= 1; }
                            continue;
                        }
                        if (!mbar_wait(&empty[astage], aphase ^ 1, abortp, wait_ns)) break;
                        mbar_expect_tx(&full[astage], kTileBytes);
                        tma_load_3d(a_ring + (size_t)astage * kTileBytes, reinterpret_cast<const CUtensorMap*>(&jb.tmap),
                                    (s.t0 + t) * 128, s.row0, s.c2, &full[astage]);
                        if (++astage == p.a_stages) { astage = 0; aphase ^= 1; }
                    }
                }
                astage = __shfl_sync(0xffffffffu, astage, 0);
                aphase = __shfl_sync(0xffffffffu, aphase, 0);
            }
        }
        // let every copy this warp issued land before the CTA's shared memory goes away:
        // the consumers wait on every full barrier they were promised, or we aborted.
    } else {
        // ------------------------------------------------------------ consumers
        const int g = lane >> 2, t4 = lane & 3;
        int astage = 0, bslot = 0;
        uint32_t aphase = 0, bphase = 0;
        for (int task = blockIdx.x; task < total && !*abortp; task += gridDim.x) {
            int j = 0, local = task;
            while (local >= cnt[j]) { local -= cnt[j]; ++j; }
            const mono_gemv_job& jb = p.a.job[j];
            const int nrb = (jb.mode == MONO_JOB_DENSE && jb.rb_per_mat > 0) ? jb.n_mats * jb.rb_per_mat : job_nrb(jb);
            int u = 0, rb, ks, nseg = 1;
            if (jb.mode == MONO_JOB_EXPERT_UP) {
                u = local / (nrb * jb.nsplit);
                local -= u * nrb * jb.nsplit;
            }
            const int u_up = u;
            rb = local % nrb;
            ks = local / nrb;
            if (jb.mode == MONO_JOB_EXPERT_DOWN) nseg = (nexp[j] > ks) ? (nexp[j] - ks + jb.nsplit - 1) / jb.nsplit : 0;

            float total_acc[NT][4];
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) total_acc[n][i] = 0.f;

            bool dead = false;
            for (int sgi = 0; sgi < nseg && !dead; ++sgi) {
                if (jb.mode == MONO_JOB_EXPERT_DOWN) u = ks + sgi * jb.nsplit;
                Seg s = make_seg<WK>(jb, rb, ks, u, nexp[j], p.bb);
                float seg_acc[NT][4];
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i) seg_acc[n][i] = 0.f;
                // weight scales of the segment: one per tile, lane i keeps tile i's
                float ws_lane = 1.f;
                if (WK == MONO_W_FP8) ws_lane = (lane < s.nt) ? __ldg(reinterpret_cast<const float*>(s.wsc) + lane) : 0.f;
                const uint8_t* ws8_g = nullptr;
                const uint8_t* ws8_g8 = nullptr;
                if (WK == MONO_W_MXFP4) {
                    int r0 = min(s.row0 - jb.row_off + warp * 16 + g, jb.n_rows - 1);
                    int r1 = min(s.row0 - jb.row_off + warp * 16 + g + 8, jb.n_rows - 1);
                    ws8_g = reinterpret_cast<const uint8_t*>(s.wsc) + (size_t)(r0 - (s.row0 - jb.row_off)) * jb.wscale_ld;
                    ws8_g8 = reinterpret_cast<const uint8_t*>(s.wsc) + (size_t)(r1 - (s.row0 - jb.row_off)) * jb.wscale_ld;
                }
                if (!mbar_wait(&bfull[bslot], bphase, abortp, wait_ns)) { dead = true; break; }
                const uint32_t slot = smem_u32(b_ring + (size_t)bslot * p.bslot_bytes);
                const uint32_t sc_base = slot + p.scale_off;

                uint2 wsn_g = make_uint2(0, 0), wsn_g8 = make_uint2(0, 0);
                if (WK == MONO_W_MXFP4) {
                    wsn_g = __ldg(reinterpret_cast<const uint2*>(ws8_g));
                    wsn_g8 = __ldg(reinterpret_cast<const uint2*>(ws8_g8));
                }
                for (int t = 0; t < s.nt; ++t) {
                    if (!mbar_wait(&full[astage], aphase, abortp, wait_ns)) { dead = true; break; }
                    const uint32_t a_base = smem_u32(a_ring + (size_t)astage * kTileBytes) + (warp * 16 + g) * 128;
                    if (WK == MONO_W_FP8 || WK == MONO_W_BF16) {
                        uint4 x0 = lds128(a_base + (((2 * t4) ^ g) << 4));
                        uint4 x1 = lds128(a_base + (((2 * t4 + 1) ^ g) << 4));
                        uint4 y0 = lds128(a_base + 1024 + (((2 * t4) ^ g) << 4));
                        uint4 y1 = lds128(a_base + 1024 + (((2 * t4 + 1) ^ g) << 4));
                        const uint32_t ar0[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                        const uint32_t ar1[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
                        float d[NT][4];
#pragma unroll
                        for (int n = 0; n < NT; ++n)
#pragma unroll
                            for (int i = 0; i < 4; ++i) d[n][i] = (WK == MONO_W_BF16) ? seg_acc[n][i] : 0.f;
                        for (int pl = 0; pl < jb.planes; ++pl) {
#pragma unroll
                            for (int n = 0; n < NT; ++n) {
                                const uint32_t b_addr = slot + (uint32_t)((pl * NPAD + n * 8 + g) * p.b_pitch) + t * 128 + 32 * t4;
                                uint4 b0 = lds128(b_addr), b1 = lds128(b_addr + 16);
                                const uint32_t br[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    if (WK == MONO_W_FP8)
                                        mma_e4m3(d[n], ar0[2 * i], ar1[2 * i], ar0[2 * i + 1], ar1[2 * i + 1], br[2 * i], br[2 * i + 1]);
                                    else
                                        mma_bf16(d[n], ar0[2 * i], ar1[2 * i], ar0[2 * i + 1], ar1[2 * i + 1], br[2 * i], br[2 * i + 1]);
                                }
                            }
                        }
                        if (WK == MONO_W_FP8) {
                            const float ws = __shfl_sync(0xffffffffu, ws_lane, t);
#pragma unroll
                            for (int n = 0; n < NT; ++n) {
                                const uint32_t sa = sc_base + (uint32_t)((n * 8 + 2 * t4) * p.scale_pitch) + t * 4;
                                const float s0 = ws * __uint_as_float(lds32(sa));
                                const float s1 = ws * __uint_as_float(lds32(sa + p.scale_pitch));
                                seg_acc[n][0] += d[n][0] * s0;
                                seg_acc[n][1] += d[n][1] * s1;
                                seg_acc[n][2] += d[n][2] * s0;
                                seg_acc[n][3] += d[n][3] * s1;
                            }
                        } else {
#pragma unroll
                            for (int n = 0; n < NT; ++n)
#pragma unroll
                                for (int i = 0; i < 4; ++i) seg_acc[n][i] = d[n][i];
                        }
                    } else {
                        // MXFP4 weights x MXFP8 activations: one MMA per 32-k scale block
                        const uint2 ws_g = wsn_g, ws_g8 = wsn_g8;
                        if (t + 1 < s.nt) {
                            wsn_g = __ldg(reinterpret_cast<const uint2*>(ws8_g + (t + 1) * 8));
                            wsn_g8 = __ldg(reinterpret_cast<const uint2*>(ws8_g8 + (t + 1) * 8));
                        }
                        uint2 as0[NT], as1[NT];
#pragma unroll
                        for (int n = 0; n < NT; ++n) {
                            const uint32_t sa = sc_base + (uint32_t)((n * 8 + 2 * t4) * p.scale_pitch) + t * 8;
                            as0[n] = lds64(sa);
                            as1[n] = lds64(sa + p.scale_pitch);
                        }
#pragma unroll
                        for (int blk = 0; blk < 8; ++blk) {
                            const uint32_t wa = lds32(a_base + ((blk ^ g) << 4) + 4 * t4);
                            const uint32_t wb = lds32(a_base + 1024 + ((blk ^ g) << 4) + 4 * t4);
                            const uint32_t a0 = fp4_lo_to_e4m3(wa), a1 = fp4_lo_to_e4m3(wb);
                            const uint32_t a2 = fp4_hi_to_e4m3(wa), a3 = fp4_hi_to_e4m3(wb);
                            const int wsg = (int)(((blk < 4 ? ws_g.x : ws_g.y) >> ((blk & 3) * 8)) & 0xFF);
                            const int wsg8 = (int)(((blk < 4 ? ws_g8.x : ws_g8.y) >> ((blk & 3) * 8)) & 0xFF);
#pragma unroll
                            for (int n = 0; n < NT; ++n) {
                                const uint32_t b_addr = slot + (uint32_t)((n * 8 + g) * p.b_pitch) + t * 256 + blk * 32 + 8 * t4;
                                const uint2 b = lds64(b_addr);
                                float d[4] = {0.f, 0.f, 0.f, 0.f};
                                mma_e4m3(d, a0, a1, a2, a3, b.x, b.y);
                                const int a_c0 = (int)(((blk < 4 ? as0[n].x : as0[n].y) >> ((blk & 3) * 8)) & 0xFF);
                                const int a_c1 = (int)(((blk < 4 ? as1[n].x : as1[n].y) >> ((blk & 3) * 8)) & 0xFF);
                                // 2^(w-127) * 2^(a-127) * 2^6
                                const float f00 = __uint_as_float((uint32_t)max(wsg + a_c0 - 121, 1) << 23);
                                const float f01 = __uint_as_float((uint32_t)max(wsg + a_c1 - 121, 1) << 23);
                                const float f10 = __uint_as_float((uint32_t)max(wsg8 + a_c0 - 121, 1) << 23);
                                const float f11 = __uint_as_float((uint32_t)max(wsg8 + a_c1 - 121, 1) << 23);
                                seg_acc[n][0] += d[0] * f00;
                                seg_acc[n][1] += d[1] * f01;
                                seg_acc[n][2] += d[2] * f10;
                                seg_acc[n][3] += d[3] * f11;
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[astage]);
                    if (++astage == p.a_stages) { astage = 0; aphase ^= 1; }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&bempty[bslot]);
                if (++bslot == p.n_bslots) { bslot = 0; bphase ^= 1; }
                // fold the segment into the task's sum (route coefficient per row of the step)
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    float c0 = 1.f, c1 = 1.f;
                    if (s.coef) { c0 = s.coef[n * 8 + 2 * t4]; c1 = s.coef[n * 8 + 2 * t4 + 1]; }
                    total_acc[n][0] += seg_acc[n][0] * c0;
                    total_acc[n][1] += seg_acc[n][1] * c1;
                    total_acc[n][2] += seg_acc[n][2] * c0;
                    total_acc[n][3] += seg_acc[n][3] * c1;
                }
            }
            if (dead) break;
            // epilogue: f32 partial sums [col][row]
            int out_row = rb * 128 + warp * 16 + g;
            int row_in_mat = (jb.mode == MONO_JOB_DENSE && jb.rb_per_mat > 0) ? (rb % jb.rb_per_mat) * 128 + warp * 16 + g
                                                                                 : out_row;
            float* out = jb.out + (size_t)((jb.mode == MONO_JOB_EXPERT_UP ? u_up * jb.nsplit : 0) + ks) * jb.out_split_stride;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const int c0 = n * 8 + 2 * t4;
                if (row_in_mat < jb.n_rows) {
                    if (c0 < p.a.rows) out[(size_t)c0 * jb.out_ld + out_row] = total_acc[n][0];
                    if (c0 + 1 < p.a.rows) out[(size_t)(c0 + 1) * jb.out_ld + out_row] = total_acc[n][1];
                }
                if (row_in_mat + 8 < jb.n_rows) {
                    if (c0 < p.a.rows) out[(size_t)c0 * jb.out_ld + out_row + 8] = total_acc[n][2];
                    if (c0 + 1 < p.a.rows) out[(size_t)(c0 + 1) * jb.out_ld + out_row + 8] = total_acc[n][3];
                }
            }
        }
    }
    __syncthreads();
    if (abort_flag) {
        // a wait ran out: give the copies still in flight time to land in this CTA's
        // shared memory before it is released, then record the failure
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        if (tid == 0 && !guard_failed(p.a.guard)) guard_fail(p.a.guard, MONO_ERR_DEADLINE, 100);
    }
}

}  // namespace mono

// ------------------------------------------------------------------------ host
extern void mono_set_error(const char* fmt, ...);
int mono_gemv_tc_enabled();                                                      // gemv_tc.cu
int mono_gemv_tc_launch(const mono_gemv_args* a, long tasks, cudaStream_t st);  // gemv_tc.cu
int mono_gemv_tc4_launch(const mono_gemv_args* a, long tasks, cudaStream_t st); // gemv_tc4.cu
int mono_gemv_tc4bs_launch(const mono_gemv_args* a, long tasks, cudaStream_t st); // gemv_tc4bs.cu
int mono_gemv_nvf4_launch(const mono_gemv_args* a, long tasks, cudaStream_t st);  // gemv_nvf4.cu
int mono_gemv_mxf4_launch(const mono_gemv_args* a, long tasks, cudaStream_t st);  // gemv_nvf4.cu (its MXFP4 instance)

namespace {
template <int WK, int NT>
int launch_gemv(const mono::GemvParams& p, int grid, size_t smem, cudaStream_t st) {
    auto k = mono::gemv_kernel<WK, NT>;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);  // 227 KB less the static part
        if (e != cudaSuccess) return (int)e;
        mono::attr_done(attr_once);
    }
    cudaError_t e = mono::launch_k(k, grid, mono::kGemvThreads, smem, st, p);
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}
}  // namespace

extern "C" int mono_gemv_launch(const mono_gemv_args* a, void* stream) {
    using namespace mono;
    if (!a || a->njobs < 1 || a->njobs > MONO_GEMV_MAX_JOBS || a->rows < 1 || a->rows > MONO_MAX_ROWS) {
        mono_set_error("mono_gemv_launch: njobs in 1..%d and rows in 1..%d required", MONO_GEMV_MAX_JOBS, MONO_MAX_ROWS);
        return MONO_E_ARG;
    }
    if (a->wkind < MONO_W_FP8 || a->wkind > MONO_W_NVFP4) {
        mono_set_error("mono_gemv_launch: unknown wkind %d", a->wkind);
        return MONO_E_ARG;
    }
    GemvParams p;
    p.a = *a;
    const int NT = a->rows > 8 ? 2 : 1, NPAD = NT * 8;
    p.bb = (a->wkind == MONO_W_MXFP4 || a->wkind == MONO_W_NVFP4) ? 256 : 128;
    int max_seg_tiles = 0, max_planes = 1;
    long tasks = 0;
    for (int j = 0; j < a->njobs; ++j) {
        const mono_gemv_job& jb = a->job[j];
        if (jb.n_rows < 1 || jb.k_tiles < 1 || jb.nsplit < 1 || jb.planes < 1 || jb.planes > 2 || !jb.act || !jb.out) {
            mono_set_error("mono_gemv_launch: job %d: bad sizes or null pointers", j);
            return MONO_E_ARG;
        }
        if (((uintptr_t)jb.act & 15) || (jb.act_ld & 15) || (jb.act_plane_stride & 15) || (jb.act_seg_stride & 15)) {
            mono_set_error("mono_gemv_launch: job %d: activation planes must be 16-byte aligned", j);
            return MONO_E_ARG;
        }
        int seg_tiles;
        if (jb.mode == MONO_JOB_EXPERT_DOWN) {
            seg_tiles = jb.k_tiles;
        } else {
            if (jb.split_tiles < 1 || (jb.nsplit > 1 && (jb.split_tiles & 3)) ||
                (long)jb.split_tiles * jb.nsplit < jb.k_tiles) {
                mono_set_error("mono_gemv_launch: job %d: split_tiles must be a multiple of 4 covering K", j);
                return MONO_E_ARG;
            }
            seg_tiles = jb.split_tiles < jb.k_tiles ? jb.split_tiles : jb.k_tiles;
        }
        if (seg_tiles > (a->wkind == MONO_W_BF16 ? 64 : 32)) {  // FP8 keeps one weight scale per lane; bf16 has none
            mono_set_error("mono_gemv_launch: job %d: a segment may span at most 32 tiles (64 for bf16), got %d", j, seg_tiles);
            return MONO_E_ARG;
        }
        if (jb.mode != MONO_JOB_DENSE && (!jb.expert_list || !jb.n_expert || jb.max_expert < 1)) {
            mono_set_error("mono_gemv_launch: job %d: expert jobs need expert_list / n_expert / max_expert", j);
            return MONO_E_ARG;
        }
        if (a->wkind == MONO_W_FP8 && (!jb.wscale_f32 || !jb.ascale_f32 || (jb.ascale_ld & 3) || ((uintptr_t)jb.ascale_f32 & 15))) {
            mono_set_error("mono_gemv_launch: job %d: FP8 jobs need f32 weight and activation scales (ld %% 4 == 0)", j);
            return MONO_E_ARG;
        }
        if (a->wkind == MONO_W_MXFP4 && (!jb.wscale_e8 || !jb.ascale_e8 || (jb.ascale_ld & 15) || ((uintptr_t)jb.ascale_e8 & 15) ||
                                         (jb.wscale_ld & 7) || ((uintptr_t)jb.wscale_e8 & 7))) {
            mono_set_error("mono_gemv_launch: job %d: MXFP4 jobs need E8M0 weight and activation scales", j);
            return MONO_E_ARG;
        }
        if (a->wkind == MONO_W_NVFP4 && (!jb.wscale_t || !jb.ascale_e8)) {
            mono_set_error("mono_gemv_launch: job %d: NVFP4 jobs need E4M3 weight and activation scale bytes", j);
            return MONO_E_ARG;
        }
        max_seg_tiles = seg_tiles > max_seg_tiles ? seg_tiles : max_seg_tiles;
        max_planes = jb.planes > max_planes ? jb.planes : max_planes;
        const int nrb = (jb.n_rows + 127) / 128;
        if (jb.mode == MONO_JOB_DENSE)
            tasks += (long)(jb.rb_per_mat > 0 ? jb.n_mats * jb.rb_per_mat : nrb) * jb.nsplit;
        else if (jb.mode == MONO_JOB_EXPERT_UP)
            tasks += (long)jb.max_expert * nrb * jb.nsplit;
        else
            tasks += (long)nrb * jb.nsplit;
    }
    if (a->wkind == MONO_W_FP8 && mono_gemv_tc_enabled()) {
        // tcgen05 path: needs the activation tensor map of every job (an all-zero map means "not given")
        bool maps = true;
        for (int j = 0; j < a->njobs; ++j) {
            const unsigned long long* w = reinterpret_cast<const unsigned long long*>(&a->job[j].act_tmap);
            unsigned long long any = 0;
            for (int i = 0; i < 16; ++i) any |= w[i];
            maps = maps && any != 0;
        }
        if (maps) {
            int rc = mono_gemv_tc_launch(a, tasks, (cudaStream_t)stream);
            if (rc > 0) mono_set_error("mono_gemv_launch: CUDA error %d (%s)", rc, cudaGetErrorString((cudaError_t)rc));
            return rc;
        }
    }
    for (int j = 0; j < a->njobs; ++j) {
        if (a->job[j].stage_planes) {
            mono_set_error("mono_gemv_launch: job %d: an output is staged by the FP8 tcgen05 path only (activation maps set)", j);
            return MONO_E_ARG;
        }
    }
    if (a->wkind == MONO_W_NVFP4) {
        // one consumer only: the block-scaled FP4 tensor-core kind takes both operands in 4 bits
        const int rc = mono_gemv_nvf4_launch(a, tasks, (cudaStream_t)stream);
        if (rc == -100) {
            mono_set_error("mono_gemv_launch: an NVFP4 job needs its weight and activation maps, one MONO_ACT_NVF4 plane, repacked weight "
                           "scales (wscale_t: whole row blocks and tiles, 16-byte aligned), row_off a multiple of 128 and segments of "
                           "at most 2048 values");
            return MONO_E_ARG;
        }
        if (rc > 0) mono_set_error("mono_gemv_launch: CUDA error %d (%s)", rc, cudaGetErrorString((cudaError_t)rc));
        return rc;
    }
    if (a->wkind == MONO_W_MXFP4 && mono_gemv_tc_enabled()) {
        // the block-scaled kind (scales read by the MMA from tensor memory): with repacked scale codes (wscale_t) the
        // kernel whose nibbles TMA pads, else (or MONO_TC4_BLOCK_SCALE=1) the one whose warps spread them;
        // MONO_TC4_BLOCK_SCALE=0 asks for the kernel that issues one MMA per scale group and scales in its epilogue
        // (read per launch: tests compare the three)
        const char* bs = getenv("MONO_TC4_BLOCK_SCALE");
        const char mode = bs ? bs[0] : '2';
        int rc = mode == '2' ? mono_gemv_mxf4_launch(a, tasks, (cudaStream_t)stream) : -100;
        if (rc == -100 && mode != '0') rc = mono_gemv_tc4bs_launch(a, tasks, (cudaStream_t)stream);
        if (rc == -100) rc = mono_gemv_tc4_launch(a, tasks, (cudaStream_t)stream);  // -100: not eligible, use the warp-MMA consumer
        if (rc != -100) {
            if (rc > 0) mono_set_error("mono_gemv_launch: CUDA error %d (%s)", rc, cudaGetErrorString((cudaError_t)rc));
            return rc;
        }
    }
    for (int j = 0; j < a->njobs; ++j) {
        if (a->wkind == MONO_W_MXFP4 && a->job[j].act_natural) {
            mono_set_error("mono_gemv_launch: job %d: natural-order MXFP8 activations need the tcgen05 path (tmap4, act_tmap, one plane, "
                           "segments of at most 2048 values)", j);
            return MONO_E_ARG;
        }
    }
    for (int j = 0; j < a->njobs; ++j) {
        if (a->job[j].feeds_job > 0) {
            mono_set_error("mono_gemv_launch: job %d: chained jobs run on the tcgen05 path only (FP8, activation maps set)", j);
            return MONO_E_ARG;
        }
    }
    // row pitch = 16 (32 for the 8-byte MXFP4 reads) mod 128: conflict-free fragment loads
    p.b_pitch = max_seg_tiles * p.bb + (a->wkind == MONO_W_MXFP4 ? 32 : 16);
    p.scale_off = max_planes * NPAD * p.b_pitch;
    p.scale_pitch = a->wkind == MONO_W_FP8 ? (((max_seg_tiles + 3) & ~3) * 4 + 16)
                                           : (a->wkind == MONO_W_MXFP4 ? (((max_seg_tiles * 8 + 15) & ~15) + 16) : 0);
    p.bslot_bytes = (p.scale_off + NPAD * p.scale_pitch + 127) & ~127;
    const int budget = 226 * 1024 - 3072;
    p.a_stages = kMaxAStages;
    while (p.a_stages > 3 && p.a_stages * kTileBytes + 2 * p.bslot_bytes > budget) --p.a_stages;
    p.n_bslots = (budget - p.a_stages * kTileBytes) / p.bslot_bytes;
    if (p.n_bslots > kMaxBSlots) p.n_bslots = kMaxBSlots;
    if (p.n_bslots < 1) {
        mono_set_error("mono_gemv_launch: activation slot of %d bytes does not fit shared memory", p.bslot_bytes);
        return MONO_E_ARG;
    }
    const size_t smem = 1024 + (size_t)p.a_stages * kTileBytes + (size_t)p.n_bslots * p.bslot_bytes + 512;
    int sms = mono_sm_count();
    if (sms <= 0) return MONO_E_DRIVER;
    int grid = a->max_ctas > 0 ? a->max_ctas : sms;
    if (grid > tasks) grid = (int)tasks;
    if (grid < 1) grid = 1;
    cudaStream_t st = (cudaStream_t)stream;
    int rc;
#define MONO_GEMV_CASE(WKC)                                                                  \
    case WKC:                                                                                \
        rc = NT == 1 ? launch_gemv<WKC, 1>(p, grid, smem, st) : launch_gemv<WKC, 2>(p, grid, smem, st); \
        break;
    switch (a->wkind) {
        MONO_GEMV_CASE(MONO_W_FP8)
        MONO_GEMV_CASE(MONO_W_MXFP4)
        MONO_GEMV_CASE(MONO_W_BF16)
        default: rc = MONO_E_ARG;
    }
#undef MONO_GEMV_CASE
    if (rc != 0) mono_set_error("mono_gemv_launch: CUDA error %d (%s)", rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "arg");
    return rc;
}
