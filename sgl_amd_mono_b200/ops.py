"""Torch-facing wrappers of the C-ABI launches: tensor checks, then pointer-only dispatch.

Mirrors the reference's operator level (``glm53/gfx950/runner.py:240-321``: shape /
dtype / contiguity checks that raise ``ValueError`` naming the tensor, then raw
pointers, scalars and the current stream go to the launcher).  All buffers are
allocated when an op is built, never during a launch, so launches are safe under
CUDA-graph capture (``deepseek_v41/gfx950/runner.py:127-132``).
"""

from __future__ import annotations

import ctypes as C
import logging
import os

import torch

from . import _lib as L

log = logging.getLogger("sgl_amd_mono_b200")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t) -> int | None:
    return None if t is None else t.data_ptr()


def _up(x: int, m: int) -> int:
    return -(-x // m) * m


def sm_count() -> int:
    """SMs of the current device (every persistent grid is sized by it: ``common/plan.py:23-25`` sizes the
    reference's by its 256 CUs).  Without a visible device (host-only planning and its CPU tests) the
    B200's count."""
    n = L.load().mono_sm_count()
    return n if n > 0 else 148


def require(t: torch.Tensor, name: str, dtype=None, shape=None, cuda: bool = True) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise ValueError(f"{name}: expected a tensor, got {type(t).__name__}")
    if cuda and not t.is_cuda:
        raise ValueError(f"{name}: must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name}: dtype {t.dtype}, needs {dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name}: shape {tuple(t.shape)}, needs {tuple(shape)}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: must be contiguous")
    return t


class ActBuf:
    """Activation planes + scales of one GEMV operand ([segs][planes][16][ld] bytes)."""

    def __init__(self, fmt: int, k: int, device, segs: int = 1):
        self.fmt, self.k, self.segs = fmt, k, segs
        self.nplanes = 2 if fmt == L.ACT_HILO else 1
        kpad = _up(k, 256)  # room for the zero tail an MXFP4 tile may read
        self.ld = 2 * kpad if fmt == L.ACT_BF16 else (kpad // 2 if fmt == L.ACT_NVF4 else kpad)
        self.planes = torch.zeros(segs, self.nplanes, L.MAX_ROWS, self.ld, dtype=torch.uint8, device=device)
        self.scale_f32 = self.scale_e8 = None
        self.scale_ld = 0
        if fmt in (L.ACT_A8, L.ACT_HILO):
            self.scale_ld = _up(kpad // 128, 4) + 4
            self.scale_f32 = torch.zeros(segs, L.MAX_ROWS, self.scale_ld, dtype=torch.float32, device=device)
        elif fmt in (L.ACT_MX8, L.ACT_MX8N):
            self.scale_ld = _up(kpad // 32, 16) + 16
            self.scale_e8 = torch.full((segs, L.MAX_ROWS, self.scale_ld), 127, dtype=torch.uint8, device=device)
        elif fmt == L.ACT_NVF4:
            # an E4M3 byte per 16 values; bytes past K stay 1.0 (0x38)
            self.scale_ld = _up(kpad // 16, 16) + 16
            self.scale_e8 = torch.full((segs, L.MAX_ROWS, self.scale_ld), 0x38, dtype=torch.uint8, device=device)

    @property
    def plane_stride(self) -> int:
        return L.MAX_ROWS * self.ld

    @property
    def seg_stride(self) -> int:
        return self.nplanes * L.MAX_ROWS * self.ld

    @property
    def scale_seg_stride(self) -> int:
        return L.MAX_ROWS * self.scale_ld


def act_prep(rows: int, k: int, dst: ActBuf | None, *, src_bf16=None, src_f32=None, nsum: int = 1,
             gamma=None, eps: float = 0.0, round_bf16: bool = True, out_bf16=None) -> None:
    """RMSNorm (optional) + quantisation of ``rows`` rows into ``dst`` (segment 0)."""
    a = L.ActPrepArgs()
    a.rows, a.k = rows, k
    a.src_bf16, a.src_f32 = _p(src_bf16), _p(src_f32)
    if src_f32 is not None:
        a.nsum, a.src_ld, a.src_sum_stride = nsum, src_f32.shape[-1], L.MAX_ROWS * src_f32.shape[-1]
    a.gamma_bf16, a.eps, a.round_bf16 = _p(gamma), eps, int(round_bf16)
    if dst is not None:
        a.fmt, a.planes, a.plane_stride, a.ld = dst.fmt, _p(dst.planes), dst.plane_stride, dst.ld
        a.scale_f32, a.scale_e8, a.scale_ld = _p(dst.scale_f32), _p(dst.scale_e8), dst.scale_ld
    a.out_bf16 = _p(out_bf16)
    L.check(L.load().mono_act_prep_launch(C.byref(a), _stream()), "mono_act_prep_launch")


_TILE_K = {L.W_FP8: 128, L.W_BF16: 64, L.W_MXFP4: 256, L.W_NVFP4: 256}
_MAX_SEG_TILES = {L.W_FP8: 16, L.W_BF16: 16, L.W_MXFP4: 8, L.W_NVFP4: 8}


def plan_split(k_tiles: int, row_blocks: int, wkind: int, sms: int | None = None, cap: int | None = None):
    """(split_tiles, nsplit): K splits of whole 4-tile groups so that row_blocks x
    nsplit tasks cover the SMs about twice and a segment fits the activation slot."""
    if cap is None and wkind == L.W_FP8:
        # the tcgen05 consumer has no activation slot to fit: segments of up to 32 tiles, fewer K splits
        lib = L.load()
        tc_on = lib.mono_set_gemv_tcgen05(1)
        lib.mono_set_gemv_tcgen05(tc_on)
        cap = 32 if tc_on else None
    cap = cap or _MAX_SEG_TILES[wkind]
    sms = sms or sm_count()
    want = max(1, -(-2 * sms // max(row_blocks, 1)))
    split = min(cap, max(4, _up(-(-k_tiles // want), 4)))
    if split >= k_tiles:
        return k_tiles, 1
    return split, -(-k_tiles // split)


def tile_nvfp4_scales(ws: torch.Tensor) -> torch.Tensor:
    """NVFP4 scale bytes [mats, rows, K/16] -> [mats, row blocks, tiles * 2048] in the order ``mono_gemv_job.wscale_t``
    describes: per (128-row block, 256-value tile) four 512-byte pieces (one per 64-value MMA), byte
    ``(r % 32) * 16 + (r // 32) * 4 + b`` of a piece = row ``r`` of the block, 16-value block ``b`` of the MMA.
    Rows and tiles are padded with 0x38 (1.0)."""
    mats, rows, kb = ws.shape
    rp, kp = _up(rows, 128), _up(kb, 16)
    pad = torch.full((mats, rp, kp), 0x38, dtype=torch.uint8, device=ws.device)
    pad[:, :rows, :kb] = ws
    # [mat, row block, r // 32, r % 32, tile, MMA, block] -> [mat, row block, tile, MMA, r % 32, r // 32, block]
    t = pad.view(mats, rp // 128, 4, 32, kp // 16, 4, 4).permute(0, 1, 4, 5, 3, 2, 6).contiguous()
    return t.view(mats, rp // 128, (kp // 16) * 2048)


def tile_mxfp4_scales(ws: torch.Tensor) -> torch.Tensor:
    """MXFP4 scale codes [mats, rows, K/32] -> [mats, row blocks, tiles * 512] (``mono_gemv_job.wscale_t``): per
    (128-row block, 128-value tile) one 512-byte block, byte ``(r % 32) * 16 + (r // 32) * 4 + g`` = row ``r`` of the
    block, 32-value group ``g`` of the tile.  Rows and tiles are padded with 127 (2^0)."""
    mats, rows, kb = ws.shape
    rp, kp = _up(rows, 128), _up(kb, 4)
    pad = torch.full((mats, rp, kp), 127, dtype=torch.uint8, device=ws.device)
    pad[:, :rows, :kb] = ws
    # [mat, row block, r // 32, r % 32, tile, group] -> [mat, row block, tile, r % 32, r // 32, group]
    t = pad.view(mats, rp // 128, 4, 32, kp // 4, 4).permute(0, 1, 4, 3, 2, 5).contiguous()
    return t.view(mats, rp // 128, (kp // 4) * 512)


def fp4_tma_ok(w: torch.Tensor) -> bool:
    """Whether a packed-nibble weight [..., N, K/2] can be read as a 4-bit tensor by TMA: K a multiple of
    128, rows a multiple of 32 bytes apart, base 32-byte aligned."""
    kb = w.shape[-1] * w.element_size()
    return w.dtype == torch.uint8 and (2 * kb) % 128 == 0 and kb % 32 == 0 and w.data_ptr() % 32 == 0 and w.is_contiguous()


class Gemv:
    """One persistent weight-streaming launch over up to four jobs (``mono_gemv_launch``)."""

    def __init__(self, wkind: int, guard: torch.Tensor | None = None, deadline_s: float = 0.0, copies: dict | None = None,
                 copy_tag=None):
        """``deadline_s``: limit of every device-side wait of the launch (0 = the library's 2 s); the
        build context's deadline, as the reference arms its waits from it (``common/guard.py:4-7,69``).
        ``copies``: where a one-time repack of this launch's weights is recorded (key tuple -> tensor)."""
        self.copies, self.copy_tag = copies, copy_tag
        self.wkind = wkind
        self.args = L.GemvArgs()
        self.args.wkind = wkind
        self.args.guard = _p(guard)
        self.args.njobs = 0
        self.args.wait_ns = int(deadline_s * 1e9)
        self._keep: list = [guard]
        self._chain_words: list = []

    def _w3(self, w: torch.Tensor, name: str) -> torch.Tensor:
        if w.dim() == 2:
            w = w.unsqueeze(0)
        if w.dim() != 3 or not w.is_contiguous() or not w.is_cuda:
            raise ValueError(f"{name}: needs a contiguous CUDA [mats, rows, K] weight")
        return w

    def add(self, name: str, w: torch.Tensor, act: ActBuf, out: torch.Tensor, *, mode: int = L.JOB_DENSE,
            wscale: torch.Tensor | None = None, n_rows: int | None = None, row_off: int = 0,
            rb_per_mat: int = 0, n_mats: int = 0, nsplit: int | None = None, split_tiles: int | None = None,
            out_slice: int = 0, expert_list=None, n_expert=None, max_expert: int = 0, coef=None,
            act_per_mat: bool = False, stage: ActBuf | None = None, wglobal: torch.Tensor | None = None) -> int:
        """Adds a job; returns the number of output slices (partial sums) it writes.  ``stage``: the
        activation buffer of the next GEMV (A8 or HILO); the job then also writes its output there,
        quantised, so that no staging launch is needed in between."""
        j = self.args.njobs
        if j >= L.GEMV_MAX_JOBS:
            raise ValueError("a launch holds at most four jobs")
        w = self._w3(w, name)
        mats, rows_total, kb = w.shape[0], w.shape[1], w.shape[2] * w.element_size()
        job = self.args.job[j]
        L.check(L.load().mono_tmap_encode(C.byref(job.tmap), w.data_ptr(), kb, rows_total, mats, kb,
                                          rows_total * kb), f"mono_tmap_encode({name})")
        k_tiles = -(-kb // 128)
        n_rows = rows_total - row_off if n_rows is None else n_rows
        job.mode, job.n_rows, job.k_tiles, job.row_off = mode, n_rows, k_tiles, row_off
        job.rb_per_mat, job.n_mats = rb_per_mat, n_mats
        nrb = (n_mats * rb_per_mat) if rb_per_mat else -(-n_rows // 128)
        if mode == L.JOB_EXPERT_DOWN:
            if k_tiles > 32:
                raise ValueError(f"{name}: a down projection spans {k_tiles} tiles, at most 32")
            job.split_tiles = k_tiles
            job.nsplit = nsplit or max(1, min(max_expert, -(-2 * sm_count() // nrb)))
        else:
            tasks_rb = nrb * (max_expert if mode == L.JOB_EXPERT_UP else 1)
            st, ns = plan_split(k_tiles, tasks_rb, self.wkind)
            job.split_tiles = split_tiles or st
            job.nsplit = nsplit or -(-k_tiles // job.split_tiles)
        if self.wkind == L.W_FP8:
            ws = require(wscale, name + ".scale", torch.float32)
            ws3 = ws if ws.dim() == 3 else ws.unsqueeze(0)
            job.wscale_f32, job.wscale_mat_stride, job.wscale_ld = ws.data_ptr(), ws3.shape[1] * ws3.shape[2], ws3.shape[2]
            if ws3.shape[2] < k_tiles or ws3.shape[1] * 128 < rows_total:
                raise ValueError(f"{name}.scale: shape {tuple(ws.shape)} does not cover the weight")
        elif self.wkind == L.W_MXFP4:
            ws = require(wscale, name + ".scale", torch.uint8)
            ws3 = ws if ws.dim() == 3 else ws.unsqueeze(0)
            if ws3.shape[2] % 8:
                # a K that ends inside a 256-value tile (TMA zero-fills the weight bytes past it): the
                # kernel reads eight scale codes per tile, so the rows are padded once with the code of 1.0
                # (the reference logs its few repacks the same way: glm53/gfx950/weights.py:207-310)
                padded = torch.full((*ws3.shape[:2], _up(ws3.shape[2], 8)), 127, dtype=torch.uint8, device=ws.device)
                padded[..., : ws3.shape[2]] = ws3
                log.info("%s.scale: padded %s -> %s (one-time repack, %d bytes)", name, tuple(ws3.shape),
                         tuple(padded.shape), padded.numel())
                ws = ws3 = padded
                self._keep.append(padded)
                if self.copies is not None:
                    self.copies["MXFP4 scale rows padded to whole tiles", self.copy_tag, name] = padded
            job.wscale_e8, job.wscale_mat_stride, job.wscale_ld = ws.data_ptr(), ws3.shape[1] * ws3.shape[2], ws3.shape[2]
        elif self.wkind == L.W_NVFP4:
            ws = require(wscale, name + ".scale", torch.uint8)
            ws3 = ws if ws.dim() == 3 else ws.unsqueeze(0)
            if act.fmt != L.ACT_NVF4:
                raise ValueError(f"{name}: NVFP4 weights take NVFP4 activations (both operands of the MMA are 4-bit)")
            if ws3.shape[1] != rows_total or ws3.shape[2] * 8 < kb:
                raise ValueError(f"{name}.scale: shape {tuple(ws.shape)} does not cover the weight (one byte per 16 values)")
            # the kernel fetches the scale bytes of a (128-row block, 256-value tile) with one bulk copy, in the order
            # the tensor core copies them to its memory: repacked once (the reference logs its few repacks the same
            # way: glm53/gfx950/weights.py:207-310)
            tiled = tile_nvfp4_scales(ws3)
            log.info("%s.scale: %s -> tiled %s (one-time repack, %d bytes)", name, tuple(ws3.shape), tuple(tiled.shape),
                     tiled.numel())
            self._keep.append(tiled)
            if self.copies is not None:
                self.copies["NVFP4 scale bytes in tensor-core order", self.copy_tag, name] = tiled
            job.wscale_e8, job.wscale_mat_stride, job.wscale_ld = ws.data_ptr(), ws3.shape[1] * ws3.shape[2], ws3.shape[2]
            job.wscale_t, job.wscale_t_mat_stride, job.wscale_t_ld = tiled.data_ptr(), tiled.shape[1] * tiled.shape[2], tiled.shape[2]
            job.k_tiles4 = -(-kb // 32)  # K in 64-value MMAs: the kernel skips the MMAs past K in the last tile
            if row_off % 128:
                raise ValueError(f"{name}: an NVFP4 job starts at a multiple of 128 rows")
            if wglobal is not None:
                require(wglobal, name + ".global_scale", torch.float32)
                if wglobal.numel() != mats:
                    raise ValueError(f"{name}.global_scale: {wglobal.numel()} values for {mats} matrices")
                job.wglobal = wglobal.data_ptr()
            self._keep.append(wglobal)
        job.act, job.planes, job.act_plane_stride, job.act_ld = _p(act.planes), act.nplanes, act.plane_stride, act.ld
        L.check(L.load().mono_tmap_encode_box(C.byref(job.act_tmap), act.planes.data_ptr(), act.ld, L.MAX_ROWS,
                                              act.segs * act.nplanes, act.ld, act.plane_stride, 16),
                f"mono_tmap_encode_box({name}.act)")
        per_seg = act_per_mat or mode == L.JOB_EXPERT_DOWN
        job.act_seg_stride = act.seg_stride if per_seg else 0
        job.ascale_f32, job.ascale_e8, job.ascale_ld = _p(act.scale_f32), _p(act.scale_e8), act.scale_ld
        job.ascale_seg_stride = act.scale_seg_stride if per_seg else 0
        job.coef = _p(coef)
        job.expert_list, job.n_expert, job.max_expert = _p(expert_list), _p(n_expert), max_expert
        out_ld = out.shape[-1]
        slice_elems = L.MAX_ROWS * out_ld
        job.out = out.data_ptr() + out_slice * slice_elems * 4
        job.out_ld, job.out_split_stride = out_ld, slice_elems
        n_slices = job.nsplit * (max_expert if mode == L.JOB_EXPERT_UP else 1)
        if out.dtype != torch.float32 or out.numel() < (out_slice + n_slices) * slice_elems:
            raise ValueError(f"{name}: output buffer holds {out.numel()} f32, needs {(out_slice + n_slices) * slice_elems}")
        job.feeds_job = 0
        if stage is not None:
            if stage.fmt not in (L.ACT_A8, L.ACT_HILO) or stage.segs != 1 or mode != L.JOB_DENSE or job.nsplit != 1:
                raise ValueError(f"{name}: only a dense job without K splits can stage its output, as A8 or HILO")
            job.stage_planes, job.stage_scale = stage.planes.data_ptr(), stage.scale_f32.data_ptr()
            job.stage_ld, job.stage_scale_ld = stage.ld, stage.scale_ld
            job.stage_fmt, job.stage_plane_stride = stage.fmt, stage.plane_stride
            self._keep.append(stage)
        job.act_natural = int(act.fmt == L.ACT_MX8N)
        if self.wkind == L.W_MXFP4 and act.fmt == L.ACT_MX8N:
            # the tcgen05 consumer reads the packed nibbles as a tensor of 4-bit elements
            L.check(L.load().mono_tmap_encode_fp4(C.byref(job.tmap4), w.data_ptr(), 2 * kb, rows_total, mats, kb, rows_total * kb),
                    f"mono_tmap_encode_fp4({name})")
            job.k_tiles4 = (2 * kb) // 128
            if row_off % 128 == 0 and os.environ.get("MONO_MXFP4_TILED_SCALES", "1") != "0":
                # the scale codes once more in the order the tensor core copies them: a tile's 512 bytes then arrive by
                # one bulk copy beside its weights (one-time repack, recorded like the reference's:
                # glm53/gfx950/weights.py:207-310)
                ws3 = ws if ws.dim() == 3 else ws.unsqueeze(0)
                tiled = tile_mxfp4_scales(ws3[..., : -(-(2 * kb) // 32)])
                log.info("%s.scale: %s -> tiled %s (one-time repack, %d bytes)", name, tuple(ws3.shape), tuple(tiled.shape),
                         tiled.numel())
                self._keep.append(tiled)
                if self.copies is not None:
                    self.copies["MXFP4 scale codes in tensor-core order", self.copy_tag, name] = tiled
                job.wscale_t, job.wscale_t_mat_stride, job.wscale_t_ld = tiled.data_ptr(), tiled.shape[1] * tiled.shape[2], tiled.shape[2]
        self._keep += [w, wscale, act, out, expert_list, n_expert, coef]
        self.args.njobs = j + 1
        return job.nsplit

    def chain(self, up_job: int, down_job: int, slots: int) -> None:
        """Job ``up_job`` (up/gate) feeds job ``down_job`` inside the launch: the CTA that finishes the
        last up task of a slot applies SwiGLU and quantises into the down job's activation buffer."""
        if self.wkind != L.W_FP8 or not 0 <= up_job < down_job < self.args.njobs:
            raise ValueError("chain: FP8 launches only, and the up job must come before the job it feeds")
        dev = next(t.device for t in self._keep if isinstance(t, torch.Tensor))
        if getattr(self, "gen", None) is None:
            self.gen = torch.zeros(2, dtype=torch.int32, device=dev)
            self.args.gen = self.gen.data_ptr()
        done = torch.zeros(slots, dtype=torch.int32, device=dev)
        ready = torch.zeros(slots, dtype=torch.int32, device=dev)
        up, dn = self.args.job[up_job], self.args.job[down_job]
        up.feeds_job, up.done, up.ready = down_job + 1, done.data_ptr(), ready.data_ptr()
        dn.ready = ready.data_ptr()
        self._keep += [done, ready]
        self._chain_words += [done, ready]

    def max_resident_ctas(self) -> int:
        """CTAs of this launch's kernel the device keeps resident (``minimax_m31/residency.py:66-85``)."""
        n = L.load().mono_gemv_max_resident_ctas(C.byref(self.args))
        if n < 0:
            L.check(n, "mono_gemv_max_resident_ctas")
        return n

    def reset_chain(self) -> None:
        """After a launch that gave up (guard error) and once the host has cleared the guard words: the
        task counters, stamps and the leave counter of the chained jobs go back to zero."""
        for t in self._chain_words:
            t.zero_()
        if getattr(self, "gen", None) is not None:
            self.gen[1] = 0

    def launch(self, rows: int) -> None:
        self.args.rows = rows
        L.check(L.load().mono_gemv_launch(C.byref(self.args), _stream()), "mono_gemv_launch")


def rowdot_args(rows: int, w: torch.Tensor, x_bf16: torch.Tensor, out: torch.Tensor, out_scale: float = 1.0) -> "L.RowdotArgs":
    a = L.RowdotArgs()
    a.rows, a.n, a.k = rows, w.shape[0], w.shape[1]
    a.w, a.w_is_f32 = w.data_ptr(), int(w.dtype == torch.float32)
    if w.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"rowdot weight dtype {w.dtype}")
    a.x_bf16, a.out, a.out_ld, a.out_scale = x_bf16.data_ptr(), out.data_ptr(), out.shape[-1], out_scale
    return a


def rowdot(rows: int, w: torch.Tensor, x_bf16: torch.Tensor, out: torch.Tensor, out_scale: float = 1.0) -> None:
    a = rowdot_args(rows, w, x_bf16, out, out_scale)
    L.check(L.load().mono_rowdot_launch(C.byref(a), _stream()), "mono_rowdot_launch")


RSAG_FROM_ROWS = 12  # the reference's switch point (minimax_m3/gfx950/layout.py:33-34)


def rsag_wanted(rows: int, n: int, world: int) -> bool:
    """Whether a step's all-reduces take the reduce-scatter + all-gather form: ``MONO_AR_RSAG=1`` asks for it from
    ``RSAG_FROM_ROWS`` rows (where the column slices divide evenly), ``MONO_AR_RSAG=always`` for every step; the
    default is the all-to-all form at every row count, which measured faster on NVSwitch (one hop; the messages of
    a 16-row step are latency-bound, not bandwidth-bound).  Same bits either way."""
    import os

    mode = os.environ.get("MONO_AR_RSAG", "0")
    if world < 2 or (n // 2) % (2 * world) or mode == "0":
        return False
    return mode == "always" or rows >= RSAG_FROM_ROWS


_injectors: dict = {}


def _injector(rank: int):
    from .common.guard import FaultInjector

    if rank not in _injectors:
        _injectors[rank] = FaultInjector(rank)
    return _injectors[rank]


def _reduce_args(rows, n, partial, nsum, out, residual, slots, peer, site, guard, deadline_s) -> "L.ReduceArgs":
    a = L.ReduceArgs()
    a.rows, a.n, a.partial, a.nsum, a.ld = rows, n, partial.data_ptr(), nsum, partial.shape[-1]
    a.sum_stride = L.MAX_ROWS * partial.shape[-1]
    a.residual, a.slots, a.out = _p(residual), _p(slots), out.data_ptr()
    a.world, a.rank = 1, 0
    if peer is not None and peer.world > 1:
        a.world, a.rank = peer.world, peer.rank
        a.peer_ptrs = peer.region_table(site).data_ptr()
        a.peer_guards = peer.guard_table.data_ptr()
        a.mc_ptr = peer.mc_region(site) if getattr(peer, "mc_region", None) is not None else 0
        a.rsag = int(rsag_wanted(rows, n, peer.world))
        a.tag, a.parity = 0, 0
        a.deadline_ns = int(deadline_s * 1e9)
    if not 0 <= site <= 254:
        raise ValueError(f"site {site}: the launch tag holds sites 0..254 (tag = epoch * 256 + site + 1)")
    a.site, a.guard = site, _p(guard)
    return a


def reduce_rows(rows: int, n: int, partial: torch.Tensor, nsum: int, out: torch.Tensor, *, residual=None,
                slots=None, peer=None, site: int = 0, guard=None, deadline_s: float = 5.0) -> None:
    """Adds the partial slices, all-reduces across ranks in rank order, adds the residual."""
    if peer is not None and peer.world > 1 and _injector(peer.rank).skip(site):
        return  # MONO_FAULT_INJECT: this rank's host skips the launch; the peers' waits at `site` run out
    a = _reduce_args(rows, n, partial, nsum, out, residual, slots, peer, site, guard, deadline_s)
    L.check(L.load().mono_reduce_launch(C.byref(a), _stream()), "mono_reduce_launch")


def logits_gather(rows: int, n_local: int, partial: torch.Tensor, nsum: int, out: torch.Tensor, *, peer=None,
                  site: int = 254, guard=None, deadline_s: float = 5.0) -> None:
    """Adds the LM head's K splits in order and gathers every rank's bf16 logits into f32 ``out``
    ``[rows, world * n_local]`` (``glm53_flash/gfx950/kernel.py:3700-3770``)."""
    a = L.LogitsGatherArgs()
    a.rows, a.n_local, a.partial, a.nsum, a.ld = rows, n_local, partial.data_ptr(), nsum, partial.shape[-1]
    a.sum_stride = L.MAX_ROWS * partial.shape[-1]
    a.out, a.out_ld = out.data_ptr(), out.shape[-1]
    a.world, a.rank = 1, 0
    if peer is not None and peer.world > 1:
        if peer.logits_table is None:
            raise ValueError("the peer buffer was built without a logits region (logits_local = 0)")
        if _injector(peer.rank).skip(site):
            return
        a.world, a.rank = peer.world, peer.rank
        a.peer_ptrs, a.peer_guards = peer.logits_table.data_ptr(), peer.guard_table.data_ptr()
        a.deadline_ns = int(deadline_s * 1e9)
    a.site, a.guard = site, _p(guard)
    L.check(L.load().mono_logits_gather_launch(C.byref(a), _stream()), "mono_logits_gather_launch")


class PendingReduce:
    """A partial-sum reduction (+ all-reduce + residual) that has not been launched: the stage that consumes its
    output launches it fused with its own norm staging (``reduce_norm``).  ``out`` is where the reduced rows
    (the new residual stream, bf16 ``[16, n]``) will be."""

    def __init__(self, rows, n, partial, nsum, out, residual, slots, peer, site, guard, deadline_s):
        self.rows, self.n, self.partial, self.nsum, self.out = rows, n, partial, nsum, out
        self.residual, self.slots, self.peer, self.site, self.guard, self.deadline_s = residual, slots, peer, site, guard, deadline_s

    def args(self) -> "L.ReduceArgs":
        return _reduce_args(self.rows, self.n, self.partial, self.nsum, self.out, self.residual, self.slots, self.peer,
                            self.site, self.guard, self.deadline_s)

    def launch(self) -> torch.Tensor:
        """On its own after all (nothing downstream to fuse with)."""
        reduce_rows(self.rows, self.n, self.partial, self.nsum, self.out, residual=self.residual, slots=self.slots,
                    peer=self.peer, site=self.site, guard=self.guard, deadline_s=self.deadline_s)
        return self.out[: self.rows]


def reduce_norm(pending: PendingReduce, dst: ActBuf | None, *, gamma=None, eps: float = 0.0, round_bf16: bool = True,
                out_bf16=None) -> torch.Tensor:
    """``pending`` and the activation staging of its output in one launch (``mono_reduce_norm_launch``): the bits of
    ``pending.launch()`` followed by ``act_prep(src_bf16=pending.out, ...)``.  Returns the reduced rows."""
    if pending.peer is not None and pending.peer.world > 1 and _injector(pending.peer.rank).skip(pending.site):
        return pending.out[: pending.rows]
    r = pending.args()
    a = L.ActPrepArgs()
    a.rows, a.k = pending.rows, pending.n
    a.gamma_bf16, a.eps, a.round_bf16 = _p(gamma), eps, int(round_bf16)
    if dst is not None:
        a.fmt, a.planes, a.plane_stride, a.ld = dst.fmt, _p(dst.planes), dst.plane_stride, dst.ld
        a.scale_f32, a.scale_e8, a.scale_ld = _p(dst.scale_f32), _p(dst.scale_e8), dst.scale_ld
    a.out_bf16 = _p(out_bf16)
    L.check(L.load().mono_reduce_norm_launch(C.byref(r), C.byref(a), _stream()), "mono_reduce_norm_launch")
    return pending.out[: pending.rows]


def sparse_mla(q, kv_pages, topk_slots, out, scratch, sm_scale: float, topk: int | None = None, staged=None) -> None:
    rows, heads = q.shape[0], q.shape[1]
    a = L.SparseMlaArgs()
    a.rows, a.heads, a.topk, a.topk_ld = rows, heads, topk or topk_slots.shape[1], topk_slots.shape[1]
    a.sm_scale = sm_scale
    a.q, a.kv_pages, a.n_pages = q.data_ptr(), kv_pages.data_ptr(), kv_pages.shape[0]
    a.topk_slots, a.out, a.scratch = topk_slots.data_ptr(), out.data_ptr(), scratch.data_ptr()
    if staged is not None:  # the merge also stages the heads' outputs for the W_UV GEMV
        d = act_heads_args(rows, heads, 512, staged)
        L.check(L.load().mono_sparse_mla_quant_launch(C.byref(a), C.byref(d), _stream()), "mono_sparse_mla_quant_launch")
        return
    L.check(L.load().mono_sparse_mla_launch(C.byref(a), _stream()), "mono_sparse_mla_launch")


def act_heads_args(rows: int, heads: int, k: int, dst: ActBuf) -> "L.ActPrepArgs":
    """The destination half of a per-head staging: segment ``head`` of ``dst`` takes vector (row, head)."""
    a = L.ActPrepArgs()
    a.rows, a.k, a.segs = rows, k, heads
    a.fmt, a.planes, a.plane_stride, a.ld = dst.fmt, _p(dst.planes), dst.plane_stride, dst.ld
    a.scale_f32, a.scale_e8, a.scale_ld = _p(dst.scale_f32), _p(dst.scale_e8), dst.scale_ld
    a.seg_stride, a.scale_seg_stride = dst.seg_stride, dst.scale_seg_stride
    return a


def act_prep_heads(rows: int, heads: int, k: int, dst: ActBuf, *, src_bf16=None, src_f32=None, nsum: int = 1,
                   round_bf16: bool = True) -> None:
    """Per-head activation sets: vector (row, head) of the source goes to segment ``head`` of ``dst``."""
    a = act_heads_args(rows, heads, k, dst)
    a.src_bf16, a.src_f32 = _p(src_bf16), _p(src_f32)
    if src_f32 is not None:
        a.nsum, a.src_ld, a.src_sum_stride = nsum, src_f32.shape[-1], L.MAX_ROWS * src_f32.shape[-1]
    a.round_bf16 = int(round_bf16)
    L.check(L.load().mono_act_prep_launch(C.byref(a), _stream()), "mono_act_prep_launch")


def mla_mid(rows: int, q_lora: int, qkv, nsum: int, w: dict, eps: float, cos, sin, positions, slots, qa: ActBuf,
            kv_pages, idx_pages, kv_out, ik=None, ik_nsum: int = 0, ik_out=None) -> None:
    a = L.MlaMidArgs()
    a.rows, a.q_lora = rows, q_lora
    a.qkv, a.nsum, a.ld, a.sum_stride = qkv.data_ptr(), nsum, qkv.shape[-1], L.MAX_ROWS * qkv.shape[-1]
    if ik is not None:
        a.ik, a.ik_nsum, a.ik_ld, a.ik_sum_stride = ik.data_ptr(), ik_nsum, ik.shape[-1], L.MAX_ROWS * ik.shape[-1]
        a.ik_norm_w, a.ik_norm_b = w["idx_k_norm_w"].data_ptr(), w["idx_k_norm_b"].data_ptr()
        a.idx_pages = idx_pages.data_ptr()
    a.q_a_norm, a.kv_a_norm, a.eps = w["q_a_norm"].data_ptr(), w["kv_a_norm"].data_ptr(), eps
    a.cos, a.sin, a.positions, a.slots = cos.data_ptr(), sin.data_ptr(), positions.data_ptr(), _p(slots)
    a.qa_planes, a.qa_plane_stride, a.qa_ld = qa.planes.data_ptr(), qa.plane_stride, qa.ld
    a.qa_scale, a.qa_scale_ld = qa.scale_f32.data_ptr(), qa.scale_ld
    a.kv_pages, a.n_pages = kv_pages.data_ptr(), kv_pages.shape[0]
    a.kv_out, a.ik_out = _p(kv_out), _p(ik_out)
    L.check(L.load().mono_mla_mid_launch(C.byref(a), _stream()), "mono_mla_mid_launch")


def q_post(rows: int, heads: int, qb, nsum: int, kv_b, kv_b_scale, cos, sin, positions, q_full,
           index_heads: int = 0, iq=None, iq_nsum: int = 0, idx_q=None) -> None:
    a = L.QPostArgs()
    a.rows, a.heads = rows, heads
    a.qb, a.nsum, a.ld, a.sum_stride = qb.data_ptr(), nsum, qb.shape[-1], L.MAX_ROWS * qb.shape[-1]
    a.kv_b, a.kv_b_scale = kv_b.data_ptr(), kv_b_scale.data_ptr()
    a.cos, a.sin, a.positions, a.q_full = cos.data_ptr(), sin.data_ptr(), positions.data_ptr(), q_full.data_ptr()
    a.index_heads = index_heads
    if index_heads:
        a.iq, a.iq_nsum, a.iq_ld, a.iq_sum_stride = iq.data_ptr(), iq_nsum, iq.shape[-1], L.MAX_ROWS * iq.shape[-1]
        a.idx_q = idx_q.data_ptr()
    L.check(L.load().mono_q_post_launch(C.byref(a), _stream()), "mono_q_post_launch")


def index_prep(rows: int, index_heads: int, iq, iq_nsum: int, cos, sin, positions, idx_q, w_proj, x_bf16, idx_w,
               out_scale: float) -> None:
    """The index queries and the index head weights (``x_bf16 @ w_proj.T * out_scale``) in one launch."""
    a = L.QPostArgs()
    a.rows, a.heads, a.index_heads = rows, 0, index_heads
    a.cos, a.sin, a.positions = cos.data_ptr(), sin.data_ptr(), positions.data_ptr()
    a.iq, a.iq_nsum, a.iq_ld, a.iq_sum_stride = iq.data_ptr(), iq_nsum, iq.shape[-1], L.MAX_ROWS * iq.shape[-1]
    a.idx_q = idx_q.data_ptr()
    d = rowdot_args(rows, w_proj, x_bf16, idx_w, out_scale)
    L.check(L.load().mono_index_prep_launch(C.byref(a), C.byref(d), _stream()), "mono_index_prep_launch")


def index_args(rows: int, index_heads: int, topk: int, idx_q, idx_w, idx_pages, page_table, positions, slots,
               scores, topk_slots, topk_pos=None, iq=None, iq_nsum: int = 0, cos=None, sin=None) -> "L.IndexArgs":
    """``iq`` (with ``cos`` / ``sin``): the q_b GEMV's partial sums of the index queries; the score launch
    then makes the queries itself (tcgen05 kernel) instead of reading ``idx_q``."""
    a = L.IndexArgs()
    if iq is not None:
        a.iq, a.iq_nsum, a.iq_ld, a.iq_sum_stride = iq.data_ptr(), iq_nsum, iq.shape[-1], L.MAX_ROWS * iq.shape[-1]
        a.cos, a.sin = cos.data_ptr(), sin.data_ptr()
    a.rows, a.index_heads, a.topk = rows, index_heads, topk
    a.idx_q, a.idx_w, a.w_ld = _p(idx_q), _p(idx_w), idx_w.shape[-1] if idx_w is not None else 0
    a.idx_pages, a.n_pages = _p(idx_pages), idx_pages.shape[0] if idx_pages is not None else 0
    a.page_table, a.pt_ld = page_table.data_ptr(), page_table.shape[-1]
    a.positions, a.slots = positions.data_ptr(), _p(slots)
    a.scores, a.score_ld = scores.data_ptr(), scores.shape[-1]
    a.topk_slots, a.topk_pos = topk_slots.data_ptr(), _p(topk_pos)
    return a


def index_score(a) -> None:
    L.check(L.load().mono_index_score_launch(C.byref(a), _stream()), "mono_index_score_launch")


def index_topk(a) -> None:
    L.check(L.load().mono_index_topk_launch(C.byref(a), _stream()), "mono_index_topk_launch")


def l2_prefetch_args(tensors, limit_bytes: int | None = None) -> "L.PrefetchArgs | None":
    """Argument block that pulls ``tensors`` (contiguous device tensors) towards L2, in order, up to ``limit_bytes``."""
    a = L.PrefetchArgs()
    left = limit_bytes
    for t in tensors:
        if t is None or a.n >= L.PREFETCH_RANGES:
            continue
        nbytes = t.numel() * t.element_size()
        if left is not None:
            nbytes = min(nbytes, left)
            left -= nbytes
        if nbytes < 16 or t.data_ptr() % 16:
            continue
        a.ptr[a.n], a.bytes[a.n] = t.data_ptr(), nbytes
        a.n += 1
    return a if a.n else None


def l2_prefetch(args: "L.PrefetchArgs") -> None:
    L.check(L.load().mono_l2_prefetch_launch(C.byref(args), _stream()), "mono_l2_prefetch_launch")


def epoch_advance(guard) -> None:
    """Adds 1 to the epoch word on the device (after the last layer of a step)."""
    L.check(L.load().mono_epoch_advance_launch(guard.data_ptr(), _stream()), "mono_epoch_advance_launch")


def guard_read(guard: torch.Tensor):
    out = (C.c_int32 * 3)()
    rc = L.load().mono_guard_read(guard.data_ptr(), C.byref(out), _stream())
    return rc, tuple(out)


def route_args(rows: int, cfg_top_k: int, route_scale: float, logits, bias, slots, ids, weights, scores,
               expert_list, n_expert, coef) -> "L.RouteArgs":
    a = L.RouteArgs()
    a.rows, a.n_experts, a.top_k, a.route_scale = rows, logits.shape[-1], cfg_top_k, route_scale
    a.logits, a.nsum, a.ld, a.sum_stride = logits.data_ptr(), 1, logits.shape[-1], 0
    a.bias, a.slots = _p(bias), _p(slots)
    a.ids, a.weights, a.scores = ids.data_ptr(), weights.data_ptr(), _p(scores)
    a.expert_list, a.n_expert, a.coef = expert_list.data_ptr(), n_expert.data_ptr(), coef.data_ptr()
    return a


def route(rows: int, cfg_top_k: int, route_scale: float, logits, bias, slots, ids, weights, scores,
          expert_list, n_expert, coef) -> None:
    a = route_args(rows, cfg_top_k, route_scale, logits, bias, slots, ids, weights, scores, expert_list, n_expert, coef)
    L.check(L.load().mono_route_launch(C.byref(a), _stream()), "mono_route_launch")


def router(dot: "L.RowdotArgs", rt: "L.RouteArgs", counter: torch.Tensor) -> None:
    """Router logits and routing in one launch; ``counter`` is one zeroed int32 word on the device."""
    L.check(L.load().mono_router_launch(C.byref(dot), C.byref(rt), counter.data_ptr(), _stream()), "mono_router_launch")


def mid_args(rows: int, inter: int, up: torch.Tensor, nsum: int, dst: ActBuf, *, n_slot=None, max_slot: int = 1,
             round_bf16: bool = False) -> "L.MidArgs":
    a = L.MidArgs()
    a.rows, a.inter, a.up, a.nsum = rows, inter, up.data_ptr(), nsum
    a.n_slot, a.max_slot = _p(n_slot), max_slot
    a.fmt, a.round_bf16 = dst.fmt, int(round_bf16)
    a.planes, a.ld = dst.planes.data_ptr(), dst.ld
    a.scale_f32, a.scale_e8, a.scale_ld = _p(dst.scale_f32), _p(dst.scale_e8), dst.scale_ld
    return a


def mid(rows: int, inter: int, up: torch.Tensor, nsum: int, dst: ActBuf, **kw) -> None:
    a = mid_args(rows, inter, up, nsum, dst, **kw)
    L.check(L.load().mono_mid_launch(C.byref(a), _stream()), "mono_mid_launch")


def mid_pair(a: "L.MidArgs", b: "L.MidArgs") -> None:
    """Two activation stages (routed experts and the shared expert) in one launch."""
    L.check(L.load().mono_mid_pair_launch(C.byref(a), C.byref(b), _stream()), "mono_mid_pair_launch")
