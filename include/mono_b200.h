/*
 * mono_b200: C ABI of the sm_100a decoder-layer kernel library.
 *
 * The reference (yuychang/sgl-amd-mono) dispatches "pointer-only" launches from its
 * host runners: torch tensors are checked in Python and the kernel receives raw
 * device pointers, a few scalars and a stream (glm53/gfx950/runner.py:240-321,
 * kernel ABI glm53/gfx950/kernel.py:369-412; minimax_m31/runner.py:145-167).  Every
 * entry point below is what a binding for that dispatch level binds: plain structs
 * of device pointers and sizes, a stream handle, an int status.  No entry point
 * blocks the host, allocates, or synchronises unless it says so.
 *
 * Status: 0 = ok; > 0 = a CUDA error code from the runtime; < 0 = MONO_E_* (bad
 * argument).  mono_last_error() returns the message of the last failure on the
 * calling thread.
 */
#ifndef MONO_B200_H
#define MONO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MONO_ABI_VERSION 1

/* Cache geometry (what SGLang owns and hands over; glm53/gfx950/kernel.py:534-548,
 * 2049-2100).  A KV page holds 64 tokens: 64 x 576 E4M3 values (512 latent + 64
 * rope) followed by 64 f32 per-token scales.  An index page holds 64 x 64 bytes of
 * packed E2M1 (128 dims) followed by 64 x 4 E8M0 codes (one per 32 dims). */
#define MONO_PAGE_TOKENS 64
#define MONO_KV_DIM 576
#define MONO_KV_PAGE_BYTES (64 * 576 + 64 * 4)
#define MONO_IDX_DIM 128
#define MONO_IDX_PAGE_BYTES (64 * 64 + 64 * 4)
#define MONO_MAX_ROWS 16 /* rows of one decode / verify step */

/* Guard words: int32[MONO_GUARD_WORDS] per rank (common/guard.py:59-60,100-241). */
#define MONO_GUARD_WORDS 16
#define MONO_GUARD_EPOCH 0
#define MONO_ERR_DEADLINE 3 /* site + 1 of the wait that ran out */
#define MONO_ERR_PEER 4     /* rank + 1 of a peer that raised its flag */
#define MONO_ERR_ARG 5      /* site + 1 of a device-side argument check */
#define MONO_GUARD_FLAGS 8  /* flag word of rank r at MONO_GUARD_FLAGS + r */

#define MONO_E_ARG (-1)
#define MONO_E_NOT_BUILT (-2)
#define MONO_E_DRIVER (-3)
#define MONO_E_GUARD (-4)

int mono_abi_version(void);
/* Programmatic dependent launch between consecutive launches of one stream (on by
 * default): each kernel lets its successor start early and waits for its predecessors
 * before touching their data, so prologues and the first weight tiles overlap the
 * previous kernel's tail.  Returns the previous setting. */
int mono_set_pdl(int on);
const char* mono_last_error(void);
/* SM count of the current device (the grid every persistent launch is sized by;
 * reference: common/plan.py:23-25 BLOCKS = 256 CUs). */
int mono_sm_count(void);
/* Kernels this library has launched in this process so far (a graph replay launches none: count an eager step). */
unsigned long long mono_launch_count(void);

/* ---- guard (common/guard.py:100-241; reads replace the reference's process kill) */
/* Copies the three error words to out[3] = {deadline, peer, arg} with a blocking
 * device-to-host copy on `stream`.  Returns MONO_E_GUARD if any is non-zero. */
int mono_guard_read(const int32_t* guard_words, int32_t out[3], void* stream);

/* ---- TMA descriptors ----------------------------------------------------------
 * A weight tensor read in place: `outer` matrices of `rows` x `inner_bytes`
 * (row-major, K contiguous), rows `row_stride_bytes` apart, matrices
 * `outer_stride_bytes` apart.  The descriptor loads 128-byte x 128-row boxes with
 * the 128-byte swizzle.  Replaces the reference's one-time tile repacks
 * (glm53/gfx950/packing.py:29-133): weights stay in SGLang's layout. */
typedef struct __attribute__((aligned(64))) mono_tmap {
    unsigned char opaque[128];
} mono_tmap_t;
int mono_tmap_encode(mono_tmap_t* out, const void* base, uint64_t inner_bytes, uint64_t rows,
                     uint64_t outer, uint64_t row_stride_bytes, uint64_t outer_stride_bytes);
/* The same with boxes of 128 bytes x `box_rows` rows (16 for the activation planes that
 * feed the tcgen05 B operand). */
int mono_tmap_encode_box(mono_tmap_t* out, const void* base, uint64_t inner_bytes, uint64_t rows, uint64_t outer,
                         uint64_t row_stride_bytes, uint64_t outer_stride_bytes, uint32_t box_rows);
/* A weight of packed 4-bit elements (two per byte, even index in the low nibble): boxes of 128
 * elements x 128 rows, which TMA writes to shared memory as 128-byte rows of 16-element groups
 * padded to 16 bytes (the layout tcgen05.mma kind::f8f6f4 reads E2M1 operands in). */
int mono_tmap_encode_fp4(mono_tmap_t* out, const void* base, uint64_t inner_elems, uint64_t rows, uint64_t outer,
                         uint64_t row_stride_bytes, uint64_t outer_stride_bytes);

/* ---- activation staging (glm53/gfx950/kernel.py:1367-1414 RMSNorm staging,
 * :1440-1466 per-128 FP8 / per-32 MXFP8 quantisation) ----------------------------
 * Activation planes feed the GEMV B operand: uint8 [planes][16][ld] plus scales.
 *   MONO_ACT_BF16   1 plane of bf16 values (ld = 2K bytes), no scales
 *   MONO_ACT_A8     1 plane E4M3, f32 scale amax/448 per 128 (kernel.py:1440-1450)
 *   MONO_ACT_HILO   2 planes E4M3 (hi, lo) of bf16 values, f32 power-of-two scale per
 *                   128: the bf16 activation exactly split for FP8 MMAs
 *   MONO_ACT_MX8    1 plane E4M3, E8M0 code per 32 (kernel.py:1452-1466), values of
 *                   each group of 8 stored as k0 k2 k4 k6 k1 k3 k5 k7 (the order the
 *                   MXFP4 weight nibbles unpack in on the warp-MMA consumer)
 *   MONO_ACT_MX8N   the same values in natural k order (the tcgen05 MXFP4 consumer)
 *   MONO_ACT_NVF4   1 plane of packed E2M1 values (two per byte, even k in the low nibble, ld >= K/2
 *                   bytes), one E4M3 scale byte per 16 values in scale_e8: scale =
 *                   E4M3(max(amax, 6 * 2^-9) / 6), value = E2M1(v / scale), both round to nearest even
 *                   (the NVFP4 consumer: both operands of the block-scaled FP4 MMA are 4-bit)
 * Rows >= `rows` of every plane stay zero. */
enum { MONO_ACT_BF16 = 0, MONO_ACT_A8 = 1, MONO_ACT_HILO = 2, MONO_ACT_MX8 = 3, MONO_ACT_MX8N = 4, MONO_ACT_NVF4 = 5 };

typedef struct mono_act_prep_args {
    int rows, k;
    /* input: exactly one of src_bf16 [rows][k] or src_f32 [nsum][16][src_ld] (summed
     * over nsum in order) */
    const void* src_bf16;
    const float* src_f32;
    int nsum, src_ld;
    long src_sum_stride;
    const void* gamma_bf16; /* RMSNorm weight [k] or NULL for no norm */
    float eps;
    int round_bf16; /* round the (normalised) value to bf16 before quantising */
    /* outputs (any may be NULL) */
    int fmt;            /* MONO_ACT_* of `planes` */
    uint8_t* planes;    /* [planes][16][ld] */
    long plane_stride;  /* bytes between planes */
    int ld;             /* bytes per row */
    float* scale_f32;   /* [16][scale_ld] */
    uint8_t* scale_e8;  /* [16][scale_ld] */
    int scale_ld;
    void* out_bf16;     /* optional second output: bf16 [16][k] plain */
    /* segments (0 or 1 = none): the source row holds `segs` vectors of k values (one per
     * head); vector s of row r goes to activation set s: planes + s * seg_stride bytes,
     * scales + s * scale_seg_stride elements */
    int segs;
    long seg_stride;
    long scale_seg_stride;
} mono_act_prep_args;
int mono_act_prep_launch(const mono_act_prep_args* a, void* stream);

/* ---- weight-streaming GEMV (glm53/gfx950/kernel.py:1061-1172 mma_units; q_a|kv_a
 * :1781-1970, q_b :2183, W_UV :3975-4123, o_proj :4125, experts :4352-5187;
 * minimax_m31/a16w4.py for MXFP4) -----------------------------------------------
 * One persistent launch walks the tasks of up to MONO_GEMV_MAX_JOBS jobs.  A task
 * is one 128-row block of a weight matrix over one K range (or, for
 * MONO_JOB_EXPERT_DOWN, over a strided group of the step's experts); partial sums
 * go to f32 buffers that the next stage adds in a fixed order. */
#define MONO_GEMV_MAX_JOBS 4
/* MONO_W_NVFP4: packed E2M1 values with one E4M3 scale byte per 16 along K (wscale_e8, [mat][row][wscale_ld],
 * repacked into the tensor core's order: wscale_t) and one f32 scale per matrix (wglobal); activations MONO_ACT_NVF4.  tcgen05 only (kind::mxf4nvf4.block_scale, 16-value blocks); k_tiles
 * counts 128-byte tiles = 256 values, as for MXFP4.  (M3.1-Flash's expert format: minimax_m31/spec.py:117-121.) */
enum { MONO_W_FP8 = 0, MONO_W_MXFP4 = 1, MONO_W_BF16 = 2, MONO_W_NVFP4 = 3 };
enum { MONO_JOB_DENSE = 0, MONO_JOB_EXPERT_UP = 1, MONO_JOB_EXPERT_DOWN = 2 };

typedef struct mono_gemv_job {
    mono_tmap_t tmap;
    mono_tmap_t act_tmap; /* activation planes as [set * planes + plane][16 rows][act_ld bytes], boxes of
                             128 B x 16 rows (tcgen05 path; mono_tmap_encode_box(..., 16)) */
    int mode;       /* MONO_JOB_* */
    int n_rows;     /* rows of W this job covers (per matrix) */
    int k_tiles;    /* K in 128-byte tiles (FP8: 128 k, BF16: 64 k, MXFP4: 256 k) */
    int split_tiles;/* dense / up: tiles per K split (multiple of 4) */
    int nsplit;     /* dense / up: K splits; down: expert groups */
    int row_off;    /* first row inside each matrix */
    int rb_per_mat; /* dense: row blocks per matrix when the job spans n_mats matrices
                       (per-head W_UV; n_rows = 128 * rb_per_mat), else 0 */
    int n_mats;     /* matrices of such a job, else 0 */
    /* weight scales */
    const float* wscale_f32;  /* FP8: [mat][row block][wscale_ld] */
    const uint8_t* wscale_e8; /* MXFP4: [mat][row][wscale_ld] */
    long wscale_mat_stride;   /* elements between matrices */
    int wscale_ld;
    /* activations */
    const uint8_t* act; /* planes [planes][16][act_ld] */
    int planes;
    long act_plane_stride;
    int act_ld;
    long act_seg_stride; /* bytes between per-matrix (dense rb_per_mat) / per-expert
                            (down) activation sets */
    const float* ascale_f32;
    const uint8_t* ascale_e8;
    int ascale_ld;
    long ascale_seg_stride; /* elements */
    const float* coef; /* down: [slot][16] route coefficient, NULL = 1 */
    /* experts of this step (device): list[0..*n_expert) */
    const int32_t* expert_list;
    const int32_t* n_expert;
    int max_expert; /* upper bound of *n_expert (grid sizing only) */
    /* output f32: dense [nsplit][16][out_ld]; up [slot][nsplit][16][out_ld];
     * down [nsplit][16][out_ld] */
    float* out;
    int out_ld;
    long out_split_stride; /* elements */
    /* Chaining inside one launch (FP8 on the tcgen05 path only; expert FFN stages of
     * glm53/gfx950/kernel.py:4352-5187, where one launch runs up, activation and down).
     * An up/gate job with feeds_job > 0 (dense, or MONO_JOB_EXPERT_UP) counts its finished
     * tasks per slot in done[slot] (slot 0 for a dense job); the CTA that finishes the last
     * task of a slot adds the K splits, applies SwiGLU (gate = rows [0, n_rows/2), up = the
     * rest), quantises per 128 values into the activation planes and scales of job
     * feeds_job - 1, zeroes done[slot] and stamps ready[slot] with the launch's generation.  The
     * fed job (a later job of the same launch) waits on that stamp, slot by slot, before it
     * reads the activations; its weight tiles are requested ahead of the wait. */
    int feeds_job;  /* 1 + index of the fed job; 0 = none */
    int32_t* done;  /* [slots] task counters, zero between launches */
    int32_t* ready; /* [slots] generation stamps; also set on the fed job */
    /* MXFP4 weights on the tcgen05 path: the weight as a tensor of packed 4-bit elements
     * (mono_tmap_encode_fp4: TMA unpacks 128-element rows into the padded 128-byte rows the MMA
     * reads) and activations in natural k order (MONO_ACT_MX8N).  Without them an MXFP4 job
     * runs on the warp-MMA consumer, which needs MONO_ACT_MX8. */
    mono_tmap_t tmap4;
    int act_natural; /* 1 = the activation planes are MONO_ACT_MX8N */
    int k_tiles4;    /* K in 128-element tiles (0 = 2 * k_tiles): exact when K ends inside a 128-byte tile.
                        NVFP4: K in 64-value MMAs (0 = 4 * k_tiles); the MMAs past K in the last tile are skipped */
    /* Optional staging of the output as the next GEMV's activations (dense jobs on the tcgen05 consumer
     * with nsplit == 1): output (row c, column n) is rounded to bf16 and written as E4M3 to
     * stage_planes[c * stage_ld + n] (MONO_ACT_HILO: high byte there, low byte stage_plane_stride
     * further), with one scale per 128 columns in stage_scale[c * stage_scale_ld + n / 128]: the bytes
     * mono_act_prep_launch writes for stage_fmt = MONO_ACT_A8 or MONO_ACT_HILO. */
    uint8_t* stage_planes;
    float* stage_scale;
    int stage_ld, stage_scale_ld, stage_fmt, stage_plane_stride;
    /* NVFP4: the f32 tensor scale of each matrix, [mat]; NULL = 1.  Applied to a task's f32 sum (before the
     * route coefficient of a down job). */
    const float* wglobal;
    /* The weight's scale bytes in the order the tensor core copies them, one piece per (128-row block, unit of
     * K): [mat][row block][unit][piece], where byte ((r % 32) * 16 + (r / 32) * 4 + b) of a 512-byte block is row r
     * of the block and scale b.  NVFP4: unit = 256 values, piece = four blocks (one per 64-value MMA, b = its
     * 16-value blocks), padding 0x38.  MXFP4: unit = 128 values, piece = one block (b = its 32-value groups),
     * padding 127.  wscale_t_ld = bytes per row block, wscale_t_mat_stride = bytes per matrix; row_off a multiple
     * of 128.  The kernel fetches a unit's scales with one bulk copy next to its weights.  Required for NVFP4;
     * for MXFP4 it selects the kernel that lets TMA pad the nibbles (else warps of the kernel gather wscale_e8). */
    const uint8_t* wscale_t;
    long wscale_t_mat_stride;
    int wscale_t_ld;
} mono_gemv_job;

typedef struct mono_gemv_args {
    int njobs;
    int rows;  /* live rows of the step (1..16) */
    int wkind; /* MONO_W_*: all jobs of one launch share it */
    int32_t* guard;
    int max_ctas; /* 0 = one per SM */
    int32_t* gen; /* chained launches: [0] generation (the last CTA to leave adds 1), [1] leave counter */
    uint64_t wait_ns; /* limit of every device-side wait of the launch (barriers, ready stamps) in
                         nanoseconds; 0 = 2 s.  A wait that runs out stores 101 in the deadline word
                         of `guard`, the launch drains and returns (common/guard.py:4-7,69 ties the
                         reference's deadline to the server's watchdog the same way). */
    mono_gemv_job job[MONO_GEMV_MAX_JOBS];
} mono_gemv_args;
int mono_gemv_launch(const mono_gemv_args* a, void* stream);
/* CTAs of this argument block's kernel that the device keeps resident at once (occupancy x SM
 * count; minimax_m31/residency.py:66-85 asks the runtime the same question for the reference's
 * FFN kernel).  A launch with chained jobs is refused when its grid exceeds this, because its CTAs
 * wait on one another (minimax_m31/runner.py:125-143).  Negative = error. */
int mono_gemv_max_resident_ctas(const mono_gemv_args* a);
/* FP8 and MXFP4 jobs run on tcgen05 MMAs with TMEM accumulators (1, default) or on warp-level
 * MMAs (0); an MXFP4 job needs tmap4 and MONO_ACT_MX8N activations for the tcgen05 consumer.
 * bf16 weights always take the warp-level consumer.  Returns the old setting. */
int mono_set_gemv_tcgen05(int on);

/* ---- small matrices on CUDA cores (router logits: minimax_m31/ffn.py:601-649 fp32
 * router; glm53/gfx950/kernel.py:4199-4330 bf16 router; indexer head weights) ------
 * out[r][n] = out_scale * sum_k x[r][k] * w[n][k]; x bf16 [16][k]; w f32 or bf16 [n][k]. */
typedef struct mono_rowdot_args {
    int rows, n, k;
    const void* w;
    int w_is_f32;
    const void* x_bf16;
    float* out;
    int out_ld;
    float out_scale;
} mono_rowdot_args;
int mono_rowdot_launch(const mono_rowdot_args* a, void* stream);

/* ---- router (glm53/gfx950/kernel.py:1575-1629 route_top8, :4199-4330;
 * minimax_m31/ffn.py:601-723) ----------------------------------------------------
 * Sums the router-logit partials, applies sigmoid, picks top_k by (score + bias)
 * with ties to the lower expert id, writes ids / weights, and builds the step's
 * distinct expert list (ascending id) with the per-(slot,row) route coefficients. */
typedef struct mono_route_args {
    int rows, n_experts, top_k;
    float route_scale;
    const float* logits; /* [nsum][16][ld] partial sums */
    int nsum, ld;
    long sum_stride;
    const float* bias;      /* [n_experts] or NULL */
    const int64_t* slots;   /* [rows] or NULL; < 0 = pad row (routes nowhere) */
    int32_t* ids;           /* out [16][top_k] (-1 on pad rows) */
    float* weights;         /* out [16][top_k] */
    float* scores;          /* out [16][n_experts] sigmoid scores (parity witness) */
    int32_t* expert_list;   /* out [rows*top_k] */
    int32_t* n_expert;      /* out [1] */
    float* coef;            /* out [rows*top_k][16] */
} mono_route_args;
int mono_route_launch(const mono_route_args* a, void* stream);
/* Router logits and routing in one launch: `d` writes the logits that `r` reads (r->logits ==
 * d->out, one partial sum); the CTA that finishes its logit columns last routes the step.
 * `counter` is one zeroed device word owned by the caller (the launch leaves it zero). */
int mono_router_launch(const mono_rowdot_args* d, const mono_route_args* r, int32_t* counter, void* stream);

/* ---- expert activation (glm53/gfx950/kernel.py:4396-4415 SiLU, :5061-5064 mid
 * re-quantisation; minimax_m31/ffn.py:849-852) -----------------------------------
 * For every (expert slot, row): adds the up/gate partial sums, mid = silu(g) * u,
 * and stages mid as the down projection's activation planes. */
typedef struct mono_mid_args {
    int rows, inter; /* inter = local intermediate size */
    const float* up;  /* [slot][nsum][16][2*inter] */
    int nsum;
    const int32_t* n_slot; /* device count of slots, or NULL -> max_slot */
    int max_slot;
    int fmt;          /* MONO_ACT_A8 | MONO_ACT_MX8 | MONO_ACT_BF16 */
    int round_bf16;
    uint8_t* planes;  /* [slot][16][ld] */
    int ld;
    float* scale_f32; /* [slot][16][scale_ld] */
    uint8_t* scale_e8;
    int scale_ld;
} mono_mid_args;
int mono_mid_launch(const mono_mid_args* a, void* stream);
/* Two activation stages in one launch (the shared expert's and the routed experts'). */
int mono_mid_pair_launch(const mono_mid_args* a, const mono_mid_args* b, void* stream);

/* ---- sparse MLA decode attention (glm53/gfx950/kernel.py:3638-3973 split,
 * :3975-4075 merge; operator level of BASELINE config 2) --------------------------
 * q bf16 [rows][heads][576]; kv_pages uint8 [pages][MONO_KV_PAGE_BYTES]; topk int32
 * [rows][topk_ld] global slots (-1 = none); out bf16 [rows][heads][512].
 * scratch: mono_sparse_mla_scratch_bytes(rows, heads, topk). */
typedef struct mono_sparse_mla_args {
    int rows, heads, topk, topk_ld;
    float sm_scale;
    const void* q;
    const uint8_t* kv_pages;
    int64_t n_pages;
    const int32_t* topk_slots;
    void* out;
    void* scratch;
    int32_t* guard;
} mono_sparse_mla_args;
size_t mono_sparse_mla_scratch_bytes(int rows, int heads, int topk);
int mono_sparse_mla_launch(const mono_sparse_mla_args* a, void* stream);
/* The same, and the merge also stages every head's 512 merged values as that head's activation set
 * of the W_UV GEMV (glm53/gfx950/kernel.py:3975-4123 merges and applies W_UV in one stage): `dst`
 * describes the destination like mono_act_prep_launch does (rows, k = 512, segs = heads, fmt, planes,
 * scales and their strides; its source fields are not read). */
int mono_sparse_mla_quant_launch(const mono_sparse_mla_args* a, const mono_act_prep_args* dst, void* stream);

/* The same attention for callers that cannot allocate device memory (this entry point
 * has no counterpart in the reference, whose runner allocates all scratch itself when
 * it is built).  Once a server has given the rest of the GPU to its KV-cache pool, a
 * late cudaMalloc may fail or stall the device, and a plugin attached after that point
 * has nowhere to get a scratch buffer from.  Here `a->scratch` is ignored: the split
 * partials go to a fixed array inside the library (about 4.3 MB, held by every GPU that
 * loads the library until the process exits).  Limits: rows <= MONO_NOALLOC_MAX_ROWS,
 * heads <= MONO_NOALLOC_MAX_HEADS, topk <= MONO_NOALLOC_MAX_TOPK; larger shapes return
 * MONO_E_ARG with a message and must use mono_sparse_mla_launch.  No cudaMalloc, cudaFree
 * or allocating library routine is called.  The first call on a device looks up the
 * array's device address (cudaGetSymbolAddress, with that device current) and caches
 * it, so make that first call before any stream capture, and before the server sizes its
 * KV-cache pool: the array comes into being when the library's device code is first loaded on
 * the GPU, and a pool sized before that would have taken the memory it needs.  All calls share the one
 * array: calls that overlap on the GPU (different streams, or different threads on one
 * device) race on it and must be serialised by the caller; the array keeps the last
 * call's partials, and nothing in it has to be cleared between calls because the merge
 * only reads what the same call's split has just written. */
#define MONO_NOALLOC_MAX_ROWS 8
#define MONO_NOALLOC_MAX_HEADS 16
#define MONO_NOALLOC_MAX_TOPK 2048
int mono_sparse_mla_launch_noalloc(const mono_sparse_mla_args* a, void* stream);

/* ---- partial-sum reduction + all-reduce + residual (glm53/gfx950/kernel.py:1631-1688
 * peer_reduce, :4125-4197, :5175-5185) -------------------------------------------
 * partial = sum over nsum slices (in order) of f32 [16][ld]; rounded to bf16; with
 * world > 1 pushed as (bf16 pair, tag) 8-byte words into every peer's buffer at
 * [parity][rank][row][col/2], polled locally until all tags match or the deadline
 * runs out, summed in rank order in f32; + residual; out bf16 [rows][n]. */
typedef struct mono_reduce_args {
    int rows, n;
    const float* partial;
    int nsum, ld;
    long sum_stride;
    const void* residual; /* bf16 [rows][n] or NULL */
    const int64_t* slots; /* [rows] or NULL: pad rows (slot < 0) contribute zeros */
    void* out;            /* bf16 [rows][n] */
    /* tensor parallel */
    int world, rank;
    const uint64_t* peer_ptrs; /* device array [world]: base of every rank's region */
    uint32_t tag;              /* launch tag; 0 = take epoch * 256 + site + 1 and parity =
                                  epoch & 1 from guard word 0 (what a CUDA graph replays) */
    int parity;
    uint64_t deadline_ns;
    int site;
    int32_t* guard;
    const uint64_t* peer_guards; /* device array [world]: every rank's guard words, or NULL */
    /* NVLS variant of the push: the multicast address of the region (the same offset in every rank's
     * buffer reaches all of them through the switch), or 0 for one st.relaxed.sys store per peer.  A rank's
     * word goes out as ONE multimem.st; the waits, the reads (this rank's own copy) and the rank-ordered
     * f32 sum are the same, so both variants give the same bits.  No reduction happens in the switch: an
     * order the hardware chooses would let routing decisions differ between ranks. */
    uint64_t mc_ptr;
    /* Reduce-scatter + all-gather form (minimax_m3/gfx950/layout.py:33-34,97-114; the reference takes it from 12
     * rows): the rank that owns a pair's column slice (n / world columns) receives the partials, sums them in rank
     * order, adds the residual and pushes the finished bf16 word to the others.  Half the bytes per link, one more
     * hop, the same bits.  Needs n / 2 divisible by 2 * world. */
    int rsag;
} mono_reduce_args;
size_t mono_reduce_peer_bytes(int rows, int n, int world);
int mono_reduce_launch(const mono_reduce_args* a, void* stream);
/* The reduction above and the activation staging of mono_act_prep_launch in ONE launch (the reference runs
 * the all-reduce, the residual add and the next RMSNorm staging inside one kernel too: glm53/gfx950/kernel.py
 * :4125-4330): `r` as for mono_reduce_launch (its output, the new residual stream, is still written to r->out);
 * `a` describes the norm and the quantised planes made from that output (a->rows == r->rows, a->k == r->n,
 * no segments; a->src_* are not read).  r->out gets the bits of mono_reduce_launch.  A cluster of up to eight
 * CTAs serves a row and adds its sum of squares in CTA order, so the normalised values may differ from
 * mono_act_prep_launch's in the last bit of the f32 reciprocal root. */
int mono_reduce_norm_launch(const mono_reduce_args* r, const struct mono_act_prep_args* a, void* stream);
/* Adds 1 to the epoch word on the device (glm53/gfx950/runner.py:209-210 advance_step). */
int mono_epoch_advance_launch(int32_t* guard, void* stream);

/* ---- weights towards L2 ahead of the stage that streams them ----
 * Nothing in the reference (its one persistent kernel overlaps a stage's loads with the stage before it by
 * construction); here consecutive stages are launches, and between two weight streams HBM is idle.  The launch only
 * issues L2 prefetch requests for the byte ranges and returns; run it on a side branch of the step's graph. */
#define MONO_PREFETCH_RANGES 8
typedef struct mono_prefetch_args {
    int n;                                /* ranges in use */
    uint64_t ptr[MONO_PREFETCH_RANGES];   /* device addresses, 16-byte aligned */
    uint64_t bytes[MONO_PREFETCH_RANGES]; /* at least 16 each; a tail shorter than 16 bytes is left out */
} mono_prefetch_args;
int mono_l2_prefetch_launch(const mono_prefetch_args* a, void* stream);

/* ---- LM-head tail: K-split sum and logits all-gather (glm53_flash/gfx950/kernel.py:3700-3770 run_head's
 * push and gather; slots by launch parity, glm53_flash/gfx950/layout.py:193-215) ------------------------
 * logits = sum over nsum slices (in order) of f32 [16][ld], this rank's n_local columns.  world == 1: the
 * f32 sums go to out[row][0..n_local).  world > 1: each pair of columns is rounded to bf16 and pushed as a
 * (bf16 pair, tag) word into every rank's logits region at [parity][row][rank * n_local / 2 + pair]; the
 * launch then waits (deadline, sticky words and peer flags as in mono_reduce_launch) for every other
 * rank's words in its own region and writes f32 out[row][src * n_local + col] for all ranks: every rank
 * ends with the same bf16-rounded logits of the whole vocabulary, widened to f32. */
typedef struct mono_logits_gather_args {
    int rows, n_local;
    const float* partial;
    int nsum, ld;
    long sum_stride;
    float* out; /* f32 [rows][out_ld], out_ld >= world * n_local */
    int out_ld;
    int world, rank;
    const uint64_t* peer_ptrs; /* device array [world]: base of every rank's logits region */
    uint32_t tag;              /* 0 = epoch * 256 + site + 1 and parity = epoch & 1 from guard word 0 */
    int parity;
    uint64_t deadline_ns;
    int site;
    int32_t* guard;
    const uint64_t* peer_guards;
} mono_logits_gather_args;
size_t mono_logits_peer_bytes(int n_local, int world);
int mono_logits_gather_launch(const mono_logits_gather_args* a, void* stream);

/* ---- attention front, after q_a|kv_a (glm53/gfx950/kernel.py:1978-2003 q_a RMSNorm,
 * :2005-2101 KV RMSNorm + k_pe RoPE + cache write, :2103-2181 index key) -----------
 * One CTA per row: adds the q_a|kv_a partial sums; q_a -> RMSNorm -> bf16 -> hi/lo
 * planes for q_b; latent -> RMSNorm -> bf16, k_pe -> interleaved RoPE -> bf16; the
 * 576 values are stored as E4M3 with the power-of-two token scale
 * 2^ceil(log2(max(amax, 1e-4) / 448)) at the row's slot (slot < 0: no write).  With
 * an indexer: index key -> LayerNorm -> RoPE on dims 0..63 -> FWHT-128 -> E2M1 with
 * one E8M0 code per 32 -> index page.  kv_out / ik_out receive the values that were
 * quantised (parity witnesses). */
typedef struct mono_mla_mid_args {
    int rows, q_lora;
    const float* qkv; /* [nsum][16][ld]: q_lora | 512 latent | 64 rope */
    int nsum, ld;
    long sum_stride;
    const float* ik; /* [ik_nsum][16][ik_ld] index-key projection, or NULL */
    int ik_nsum, ik_ld;
    long ik_sum_stride;
    const void* q_a_norm;  /* bf16 [q_lora] */
    const void* kv_a_norm; /* bf16 [512] */
    float eps;
    const float* ik_norm_w; /* f32 [128] */
    const float* ik_norm_b;
    const void* cos; /* bf16 [max_pos][32] */
    const void* sin;
    const int64_t* positions;
    const int64_t* slots;
    uint8_t* qa_planes; /* hi/lo planes [2][16][qa_ld] */
    long qa_plane_stride;
    int qa_ld;
    float* qa_scale; /* [16][qa_scale_ld] */
    int qa_scale_ld;
    uint8_t* kv_pages;
    uint8_t* idx_pages;
    int64_t n_pages;
    void* kv_out;  /* bf16 [16][576] */
    float* ik_out; /* f32 [16][128] */
} mono_mla_mid_args;
int mono_mla_mid_launch(const mono_mla_mid_args* a, void* stream);

/* ---- q after q_b (glm53/gfx950/kernel.py:2183-2353 q_b + RoPE + index q, :2355-2443
 * W_UK absorb) ---------------------------------------------------------------------
 * Adds the q_b partial sums; per head: q_nope -> bf16 -> q_lat = W_UK^T q_nope (kv_b
 * rows [h*256, h*256+128) as block-FP8) -> bf16; q_pe -> RoPE -> bf16; q_full bf16
 * [16][heads][576] = q_lat | q_pe.  Index queries: RoPE on dims 0..63, FWHT-128, bf16. */
typedef struct mono_q_post_args {
    int rows, heads;
    const float* qb; /* [nsum][16][ld], per head 128 nope + 64 rope */
    int nsum, ld;
    long sum_stride;
    const uint8_t* kv_b;     /* E4M3 [heads*256][512] */
    const float* kv_b_scale; /* [heads*2][4] */
    const void* cos;
    const void* sin;
    const int64_t* positions;
    void* q_full; /* bf16 [16][heads][576] */
    int index_heads;
    const float* iq; /* [iq_nsum][16][iq_ld] or NULL */
    int iq_nsum, iq_ld;
    long iq_sum_stride;
    void* idx_q; /* bf16 [16][index_heads][128] */
} mono_q_post_args;
int mono_q_post_launch(const mono_q_post_args* a, void* stream);
/* The index queries of mono_q_post_launch (heads ignored) and a row-dot (mono_rowdot_args: the index head weights,
 * x @ weights_proj, glm53/gfx950/kernel.py:1781-1970) in one launch: the two inputs of the score launch that are still
 * missing when the q_b projection ends (kernel.py:2262-2353).  mono_rowdot_args is declared further down. */
struct mono_rowdot_args;
int mono_index_prep_launch(const mono_q_post_args* q, const struct mono_rowdot_args* d, void* stream);

/* ---- lightning indexer (glm53/gfx950/kernel.py:2684-3000 scores, :3002-3636 exact
 * top-k; FP4 keys as deepseek_v4/gfx950/kernels/stages/indexer.py:143-151) ----------
 * score[row][pos] = sum_h relu(q_h . key_pos) * w_h for pos <= positions[row], keys
 * read through the row's page-table row.  Then the exact top-k of each row: radix
 * select on the monotone image of the f32 bits, ties to the lowest position, output
 * [keys above the threshold in position order] ++ [first ties in position order],
 * published as global KV slots page * 64 + pos % 64 (-1 fills the tail; rows with at
 * most topk keys keep every key in order; pad rows get -1 everywhere). */
typedef struct mono_index_args {
    int rows, index_heads, topk;
    const void* idx_q;  /* bf16 [16][index_heads][128] */
    const float* idx_w; /* f32 [16][w_ld] */
    int w_ld;
    const uint8_t* idx_pages;
    int64_t n_pages;
    const int32_t* page_table; /* [rows][pt_ld] */
    int pt_ld;
    const int64_t* positions;
    const int64_t* slots;
    float* scores; /* [16][score_ld] */
    int score_ld;
    int32_t* topk_slots; /* [16][topk] */
    int32_t* topk_pos;   /* [16][topk] positions (parity witness) or NULL */
    /* Optional (tcgen05 score kernel only): with iq set the score launch makes the index queries itself
     * from the q_b GEMV's partial sums (sum of iq_nsum slices, interleaved RoPE on the first 64 dims,
     * orthonormal Hadamard over 128: glm53/gfx950/kernel.py:2262-2353, the index half of
     * mono_q_post_launch) and, when idx_q is not NULL, also writes them there. */
    const float* iq; /* [iq_nsum][16][iq_ld] */
    int iq_nsum, iq_ld;
    long iq_sum_stride;
    const void* cos; /* bf16 [positions][32] */
    const void* sin;
} mono_index_args;
int mono_index_score_launch(const mono_index_args* a, void* stream);
int mono_index_topk_launch(const mono_index_args* a, void* stream);

/* ---- symmetric peer memory (common/peer.py:33-64 HIP IPC calls, :118-165 PeerBuffer) --
 * A rank allocates one zeroed device buffer, exports a 64-byte handle that travels over
 * the host-side handshake (gloo), and opens every peer's handle; the opened addresses
 * are what in-kernel pushes store to.  These five calls are the only ones that allocate
 * or map memory, and they run at build time, never inside a step. */
#define MONO_IPC_HANDLE_BYTES 64
int mono_peer_alloc(size_t bytes, void** out_ptr);
int mono_peer_export(void* ptr, unsigned char handle[MONO_IPC_HANDLE_BYTES]);
int mono_peer_open(const unsigned char handle[MONO_IPC_HANDLE_BYTES], void** out_ptr);
int mono_peer_close(void* opened_ptr);
int mono_peer_free(void* ptr);
/* Blocking copy of device bytes (a peer buffer's words) to the host: for tests and post-mortems that read the
 * (value, tag) words a step left behind (the reference's layer checks read its symmetric buffer the same way,
 * test/kernels/glm53/check_layer.py:400-430). */
int mono_peer_read(void* dst_host, const void* src_device, size_t bytes);

/* ---- GQA block-sparse decode attention (minimax_m3/gfx950: pre_attn.py:8-19 head norms,
 * RoPE and cache insert; index_score.py:1-12 block scores; post_attn.py:466-592 and
 * select.py:1-56 block selection; post_attn.py:706-979 split and merge) -------------
 * Head dim 128; a block is one 64-token page; 16 blocks are attended.  K and V caches hold
 * E4M3 bytes of value / scale with the layer's fixed scalar scales, laid out
 * [page][64][kv_heads][128]; the index cache holds E4M3 index keys [page][64][128].
 * The four launches share one argument block:
 *   front   sums the fused-projection partials (q heads | k heads | v heads | index q | index k),
 *           applies the per-head Gemma RMSNorm (weight 1 + g) and the NeoX rotation of dims
 *           (i, i + 32), i < 32, writes q / index q as bf16 and inserts K, V and the index key at
 *           slots[row] (a negative slot inserts nothing);
 *   score   scores[row][b] = max over block b's causal keys of index_q . index_k, times
 *           fp32(sm_scale * log2 e);
 *   select  a context of at most 16 blocks keeps them all in order; otherwise the 16 best by
 *           (key, block id) descending, the first init_blocks pinned to 1e30 and the last
 *           local_blocks to 1e29, rank by counting; full blocks in rank order, the tail block last;
 *   attn    softmax((q . k) k_scale sm_scale) v v_scale over the selected keys: one partial per
 *           (row, kv head, slot), then a merge. */
typedef struct mono_gqa_args {
    int rows, q_heads, kv_heads;
    const float* qkv; /* [nsum][16][ld] f32 */
    int nsum, ld;
    long sum_stride;
    const void* g_q;  /* bf16 [128] each */
    const void* g_k;
    const void* g_iq;
    const void* g_ik;
    float eps;
    const void* cos; /* bf16 [positions][32] */
    const void* sin;
    const int64_t* positions; /* [rows]; the row's context is positions[row] + 1 keys */
    const int64_t* slots;     /* [rows] cache slot = page * 64 + offset, negative = pad row; may be NULL */
    float k_scale, v_scale;
    uint8_t* k_cache;
    uint8_t* v_cache;
    uint8_t* index_cache;
    int64_t n_pages;
    void* q_out;  /* bf16 [16][q_heads][128] */
    void* iq_out; /* bf16 [16][128] */
    const int32_t* page_table; /* [rows][pt_ld] page of each block */
    int pt_ld;
    float* scores; /* [16][score_ld] */
    int score_ld;
    int init_blocks, local_blocks;
    int32_t* sel_pages;  /* [16][16], -1 = empty slot */
    int32_t* sel_blocks; /* [16][16] */
    int32_t* n_ctx;      /* [16] keys attended */
    float sm_scale;
    float* scratch; /* mono_gqa_scratch_bytes(rows, q_heads) */
    void* out;      /* bf16 [16][q_heads * 128] */
} mono_gqa_args;
size_t mono_gqa_scratch_bytes(int rows, int q_heads);
int mono_gqa_front_launch(const mono_gqa_args* a, void* stream);
int mono_gqa_score_launch(const mono_gqa_args* a, void* stream);
int mono_gqa_select_launch(const mono_gqa_args* a, void* stream);
int mono_gqa_attn_launch(const mono_gqa_args* a, void* stream);

/* sizeof() of the argument structs, by index (0 gemv_job, 1 gemv_args, 2 act_prep,
 * 3 route, 4 mid, 5 sparse_mla, 6 reduce, 7 rowdot, ..., 11 gqa, 12 logits_gather): lets a binding check its mirror. */
size_t mono_struct_size(int which);

#ifdef __cplusplus
}
#endif
#endif /* MONO_B200_H */
