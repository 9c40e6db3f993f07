"""Python faces of the CUDA kernels: check sizes, pass pointers, launch on torch's current stream.

Every function refuses what its kernel cannot take with `Unsupported` (never a wrong result) and
raises `EngineError` when a launch fails. Tensors must live on the CUDA device; there is no CPU path.
"""

from __future__ import annotations

import contextlib
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from ..errors import EngineError, InvalidArgument, Unsupported
from . import lib as _lib

DL_ERR_UNSUPPORTED = 10001

_P, _I, _F, _L = c_void_p, c_int, c_float, c_longlong

# library -> function -> argument types
_SIGNATURES = {
    "embedding": {"dl_embed": [_I, _P, _P, _P, _I, _I, _I, _F, _P]},
    "norm": {
        "dl_rmsnorm": [_I, _I, _P, _P, _F, _P, _F, _P, _P, _I, _I, _I, _I, _L, _P, _L, _P],
        "dl_residual_add": [_I, _P, _P, _F, _L, _I, _L, _P],
        "dl_rmsnorm_pair": [_I, _P, _P, _I, _I, _L, _P, _I, _I, _L, _P, _P, _F, _P, _P, _P, _I, _I, _I, _P],
    },
    "activation": {"dl_silu_mul": [_I, _P, _P, _I, _I, _P], "dl_relu2": [_I, _P, _P, _L, _P],
                   "dl_gelu_tanh": [_I, _P, _P, _L, _P]},
    "norm_after_sum": {
        "dl_norm_after_sum": [_I, _I, _P, _P, _I, _L, _P, _F, _P, _F, _P, _I, _I, _P],
        "dl_cast_rows": [_I, _P, _P, _L, _P]},
    "ssm": {
        "dl_ssm_conv": [_I, _P, _I, _I, _I, _P, _P, _I, _P, _L, _L, _P, _P, _P, _P, _P, _I, _P],
        "dl_short_conv": [_I, _P, _I, _I, _I, _P, _P, _I, _P, _L, _L, _P, _P, _P, _P, _P, _I, _I, _P, _P],
        "dl_ssm_conv_keep": [_I, _P, _I, _I, _I, _I, _P, _L, _L, _P, _P, _I, _P],
        "dl_ssm_scan": [_I, _P, _I, _P, _I, _I, _P, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _I, _P, _I, _P,
                        _P, _P],
        "dl_gated_group_norm": [_I, _P, _P, _I, _P, _F, _P, _I, _I, _I, _P]},
    "latent_attention": {
        "dl_latent_prep": [_I, _P, _I, _I, _I, _I, _I, _P, _P, _F, _P, _P, _P, _P, _I, _I, _P, _P, _I, _P],
        "dl_rotate_pairs": [_I, _P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _P, _P, _I, _I, _P],
        "dl_head_linear": [_I, _P, _I, _I, _I, _P, _I, _P, _I, _I, _P, _I, _I, _I, _I, _P],
        "dl_latent_attention": [_I, _P, _I, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P]},
    "head_linear_tc": {
        "dl_head_linear_tc": [_P, _I, _I, _I, _P, _I, _P, _I, _I, _P, _I, _I, _I, _I, _P]},
    "latent_attention_flash": {
        "dl_latent_attention_flash": [_P, _I, _P, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P, _I, _I, _P,
                                      _P]},
    "qk_norm_cache": {
        "dl_qk_norm_cache_write": [_I, _P, _I, _P, _P, _P, _I, _P, _L, _I, _I, _P, _P, _F, _F, _I, _I, _I, _I, _I, _I,
                                   _I, _I, _P]},
    "attention_diff_flash": {
        "dl_diff_attention_prefill": [_P, _I, _P, _L, _I, _I, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _F, _P, _F, _F,
                                      _P],
        "dl_diff_attention_decode": [_P, _I, _P, _L, _I, _I, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _F, _P,
                                     _F, _F, _I, _P]},
    "attention_diff": {
        "dl_diff_attention": [_I, _P, _I, _P, _L, _I, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _F, _P,
                              _F, _F, _P]},
    "rope_cache": {
        "dl_rope_cache_write": [_I, _P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _F, _I, _I, _I, _I, _I, _I, _P],
        "dl_rope_angles": [_P, _P, _I, _F, _I, _P, _P]},
    "attention_generic": {
        "dl_paged_attention_generic": [_I, _P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P],
        "dl_paged_attention_generic_kv": [_I, _P, _I, _P, _L, _P, _L, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I,
                                          _P],
        "dl_paged_attention_generic_masked": [_I, _P, _I, _P, _L, _P, _L, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F,
                                              _I, _I, _I, _P]},
    "delta_rule": {
        "dl_delta_rule": [_I, _P, _I, _I, _I, _I, _P, _I, _I, _I, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "dl_delta_rule_step": [_I, _P, _I, _I, _I, _I, _P, _I, _I, _I, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "dl_head_norm_gate": [_I, _P, _P, _I, _I, _P, _F, _P, _I, _I, _I, _P]},
    "rglru": {
        "dl_rglru_gates": [_I, _P, _P, _P, _P, _P, _P, _F, _P, _P, _I, _I, _I, _P],
        "dl_rglru_scan": [_I, _P, _P, _P, _I, _I, _P, _P, _L, _P, _P, _P, _I, _I, _I, _P]},
    "qk_proj_norm": {
        "dl_qk_proj_norm_cache": [_I, _P, _I, _P, _P, _F, _I, _P, _I, _F, _P, _P, _P, _I, _P, _L, _P, _L, _I, _I, _I, _I,
                                  _I, _I, _P],
        "dl_qk_rot_head_norm_cache": [_I, _P, _I, _P, _P, _I, _I, _I, _F, _P, _P, _P, _I, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I,
                                      _P]},
    "attention_masked_flash": {
        "dl_masked_flash_attention": [_P, _I, _P, _L, _P, _L, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _I, _I, _P,
                                      _P]},
    "layer_norm": {
        "dl_stream_layer_norm": [_I, _I, _P, _I, _I, _P, _P, _I, _L, _F, _P, _P, _P, _P, _P, _F, _P, _P, _I, _I, _P],
        "dl_stream_sum": [_I, _P, _I, _I, _P, _I, _L, _F, _P, _P, _P, _I, _P]},
    "gla": {
        "dl_gla_decay": [_P, _I, _I, _I, _P, _F, _P],
        "dl_gla_scan": [_I, _P, _I, _I, _I, _I, _P, _I, _F, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P]},
    "moe": {
        "dl_moe_route": [_P, _I, _I, _I, _I, _I, _I, _F, _P, _P, _P],
        "dl_moe_group": [_P, _I, _I, _P, _P, _P, _P, _I, _P],
        "dl_moe_linear": [_I, _I, _P, _I, _P, _I, _P, _I, _I, _P, _I, _P, _P, _I, _I, _I, _I, _P],
        "dl_moe_gather": [_P, _I, _P, _I, _P, _I, _I, _P],
        "dl_moe_combine": [_I, _P, _I, _P, _P, _I, _P, _I, _P]},
    "gates": {
        "dl_gelu_mul": [_I, _P, _P, _I, _I, _P],
        "dl_sigmoid_gate": [_I, _P, _I, _P, _I, _I, _I, _P],
        "dl_scaled_sum": [_I, _P, _I, _L, _F, _I, _P, _I, _L, _F, _P, _L, _P],
        "dl_softcap": [_P, _L, _F, _P],
        "dl_add_bias": [_I, _P, _L, _P, _I, _I, _P]},
    "norm_sandwich": {
        "dl_norm_add_norm": [_I, _I, _P, _P, _I, _L, _P, _F, _P, _F, _P, _I, _I, _P]},
    "attention_decode": {
        "dl_paged_attention_decode": [_I, _P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
        "dl_paged_attention_decode_planned": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P,
                                              _I, _I, _P, _L, _P],
        "dl_paged_attention_decode_tc": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P, _L, _P]},
    "attention_prefill": {
        "dl_paged_attention_prefill": [_P, _I, _P, _P, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _P]},
    "attention_prefill_tcgen05": {
        "dl_paged_attention_prefill_tcgen05": [_P, _I, _I, _P, _P, _L, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P,
                                               _P, _P, _I, _P]},
    "gemm_skinny": {
        "dl_gemm_skinny": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _L, _P, _L, _P],
        "dl_gemm_skinny_qkv_rope": [_P, _I, _P, _P, _I, _I, _I, _P, _P, _P, _I, _P, _P, _P, _F, _I, _I, _I, _I, _P]},
    "gemm_tcgen05": {
        "dl_gemm_tcgen05": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P],
        "dl_gemm_tcgen05_tile_coords": [_I, _I, _I, _I, _P, _P],
        "dl_gemm_tcgen05_grouped": [_P, _I, _I, _P, _I, _I, _I, _P, _I, _I, _P, _P, _I, _P, _P],
        "dl_gemm_tcgen05_qkv_rope": [_P, _I, _P, _P, _I, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P, _F, _I, _I, _I, _I, _P, _P]},
    "gemm_tcgen05_cluster": {
        "dl_gemm_tcgen05_cluster": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P],
        "dl_gemm_tcgen05_cluster_qkv_rope": [_P, _I, _P, _P, _I, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P, _F, _I, _I, _I, _I, _P, _P]},
    "gemm_stream_tcgen05": {
        "dl_gemm_stream": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _L, _P, _P]},
    "gemm_simt": {"dl_gemm_simt": [_I, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _P]},
    "sampling": {
        "dl_argmax": [_P, _I, _I, _I, _P, _P, _P, _P, _P],
        "dl_sample_temperature": [_P, _I, _I, _I, _P, _P, _P, _P, _P],
        "dl_apply_penalties": [_P, _I, _I, _P, _P, _I, _P, _P, _I, _P, _P, _P],
        "dl_sample_filtered": [_P, _I, _I, _P, _I, _P, _P, _P, _P],
        "dl_argmax_of_parts": [_P, _P, _I, _I, _P, _P, _P, _P],
        "dl_feedback_tokens": [_P, _P, _P, _I, _P],
    },
    "streams": {"dl_stream_fork": [_P, _P], "dl_stream_join": [_P, _P]},
    "table_update": {"dl_table_updates": [_P, _P, _I, _I, _I, _I, _P],
                     "dl_zero_pages": [_P, _L, _I, _I, _P, _I, _I, _P]},
}

_funcs = {}


_recording: Optional[list] = None

# The checked build of the kernels (DYNALM_CHECK=1, csrc/check.cuh): every index a kernel takes from device memory
# is compared with its range before use; after every launch the host reads the library's record of the first
# violation and raises EngineError. Steps then run launch by launch (no CUDA graphs), each launch followed by a
# wait for its stream: a build for finding faults, not for speed.
CHECKED = bool(_lib.extra_flags())

CHECK_CODES = {
    1: "a token id outside the vocabulary",
    2: "a gathered row outside the rows of the step",
    3: "a request index outside the block table",
    4: "a position whose block lies outside the request's row of the block table",
    5: "a page id outside the pool",
    6: "a place outside the array of chosen ids",
    7: "a query tile whose rows lie outside the step",
    8: "a part of a query tile outside its parts, or its records outside the scratch",
}


def decode_check_record(record) -> str:
    """The sentence for a record of csrc/check.cuh: (code, value, lowest allowed, one past the highest allowed,
    blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x); '' when the code is 0."""
    code, value, lo, hi, bx, by, bz, tx = (int(v) for v in record)
    if code == 0:
        return ""
    what = CHECK_CODES.get(code, f"check code {code}")
    return f"{what}: {value} is not in [{lo}, {hi}) (block {bx},{by},{bz}, thread {tx})"


def _checked(library: str, name: str, f):
    take = getattr(_lib.load(library), "dl_check_take")
    take.argtypes = [c_void_p, c_void_p]
    take.restype = c_int
    record = (c_longlong * 8)()

    def call(*args):
        code = f(*args)
        if code != 0:
            return code
        rc = take(record, _stream())
        if rc != 0:
            raise EngineError(f"{name}: CUDA error {rc} after the launch")
        if record[0] != 0:
            raise EngineError(f"{name} (checked build): {decode_check_record(record)}; the access was not made")
        return 0
    return call


def check_limits(library: str, pages: int = 0, requests: int = 0, rows: int = 0, vocab: int = 0) -> None:
    """In a checked build: the ranges that the kernels of `library` compare their indices with from now on (in
    stream order); 0 = not known, not checked. Nothing otherwise."""
    if not CHECKED:
        return
    f = _funcs.get(("limits", library))
    if f is None:
        f = getattr(_lib.load(library), "dl_check_limits")
        f.argtypes = [_I, _I, _I, _I, _P]
        f.restype = c_int
        _funcs[("limits", library)] = f
    code = f(int(pages), int(requests), int(rows), int(vocab), _stream())
    if code != 0:
        raise EngineError(f"dl_check_limits of {library}: CUDA error {code}")


def _fn(library: str, name: str):
    f = _funcs.get(name)
    if f is None:
        f = getattr(_lib.load(library), name)
        f.argtypes = _SIGNATURES[library][name]
        f.restype = c_int
        if CHECKED and library != "streams":
            f = _checked(library, name, f)
        _funcs[name] = f
    if _timing is not None:
        return _timing.timed(name, f)
    if _recording is None:
        return f
    calls = _recording

    def recorded(*args):
        calls.append((f, args))
        return f(*args)
    return recorded


@contextlib.contextmanager
def on_stream(handle: int):
    """Inside the block every launch of this module goes to the stream with this handle."""
    global _pinned_stream
    previous = _pinned_stream
    _pinned_stream = int(handle)
    try:
        yield
    finally:
        _pinned_stream = previous


def counts_as_kernel(f) -> bool:
    """Whether a recorded function launches a kernel of this package (a library product and the ordering of two
    streams do not)."""
    return f is not library_mm_again and f is not _funcs.get("dl_stream_fork") and f is not _funcs.get("dl_stream_join")


def stream_fork(side: int) -> None:
    """What the stream `side` is given from now on runs after everything the current stream has been given so far
    (csrc/streams.cu)."""
    code = _fn("streams", "dl_stream_fork")(_stream(), int(side))
    if code != 0:
        raise EngineError(f"stream_fork: CUDA error {code}")


def stream_join(side: int) -> None:
    """What the current stream is given from now on runs after everything `side` has been given so far."""
    code = _fn("streams", "dl_stream_join")(_stream(), int(side))
    if code != 0:
        raise EngineError(f"stream_join: CUDA error {code}")


def library_mm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = x w^T by the library (cuBLAS through torch), written down like a launch of this module's when a
    recording is on."""
    if _timing is not None:
        _timing.timed("library product (torch.mm)", library_mm_again)(x, w, out)
        return
    torch.mm(x, w.t(), out=out)
    if _recording is not None:
        _recording.append((library_mm_again, (x, w, out)))


def note_unrecorded_work() -> None:
    """For device work that is not written down while a recording is on: marks the recording as incomplete, so
    that nobody repeats it."""
    if _recording is not None:
        _recording.append((None, ()))


def library_mm_again(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> int:
    torch.mm(x, w.t(), out=out)
    return 0


_timing: Optional["KernelTimes"] = None

# What the next weight-streaming kernel but one will read (see `stream_ahead`): (address, bytes) or None.
_ahead: Optional[tuple] = None
AHEAD = os.environ.get("DYNALM_AHEAD", "1") != "0"
# At most this many bytes of a hint are requested. Measured on B200 (1B shapes, decode step at batch 8 / batch 1):
# without 0.945 / 0.778 ms; 4 MB 0.934 / 0.776; 12 MB 0.912 / 0.756; 16 MB 0.920; 24 MB 0.921 / 0.759; 34 MB 0.929 / 0.780;
# everything (the 67 MB of gate | up included) 0.984 / 0.810: what is requested too early is pushed out of L2 again by
# the kernels in between and is read twice.
AHEAD_MAX = int(os.environ.get("DYNALM_AHEAD_MAX", str(12 << 20)))


def stream_ahead(weights: Optional[torch.Tensor]) -> None:
    """Says that `weights` will be streamed from memory by a kernel soon. The next kernel launched through this
    module that can do so (the norm, the decode attention, the weight-streaming products for few rows) asks for them
    to be brought into L2 before it waits for the kernel in front of it: while that kernel is still running, the
    weights of the kernel after the next already cross the memory bus, which otherwise idles at every seam between
    two short kernels of a decode step. One hint is taken by one launch; a hint nobody takes is dropped by the next
    launch that cannot. DYNALM_AHEAD=0 turns it off."""
    global _ahead
    _ahead = None if (weights is None or not AHEAD) else (weights.data_ptr(), min(AHEAD_MAX, weights.numel() * weights.element_size()))


def _take_ahead():
    global _ahead
    got, _ahead = _ahead, None
    return got if got is not None else (None, 0)


class KernelTimes:
    """Inside the block every kernel launch of this module stands between two CUDA events on its stream;
    `totals()` then gives {C entry point: (launches, milliseconds)}. A kernel launched to start beside the end of
    the one in front of it (programmatic dependent launch, on by default for the products and the attention) lets the
    event behind it pass early: run with DYNALM_PDL=0 for times that are each kernel's own. The counterpart of the reference's per-op marks
    in its forward pass (`ForwardProfile`, dynalm/src/model/transformer.h:34-49): off unless asked for, and meant
    for steps that run launch by launch (engine/profile.py sees to that)."""

    def __enter__(self):
        global _timing
        self.marks: list = []
        self._outer = _timing
        _timing = self
        return self

    def __exit__(self, *exc):
        global _timing
        _timing = self._outer
        return False

    def timed(self, name: str, f):
        def call(*args):
            # the stream the launch goes to, as a torch stream: torch's own current stream where that is it (an external
            # handle of the default stream is not the same stream to torch, and events recorded there wait for nothing)
            current = torch.cuda.current_stream()
            stream = current if current.cuda_stream == _stream() else torch.cuda.ExternalStream(_stream())
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            code = f(*args)
            end.record(stream)
            self.marks.append((name, begin, end))
            return code
        return call

    def totals(self) -> dict:
        torch.cuda.synchronize()
        out: dict = {}
        for name, begin, end in self.marks:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + begin.elapsed_time(end))
        return out


class Recording:
    """Inside the block every kernel launch of this module is also written down as (function, arguments), in
    order: `calls`; a function returns 0 when its launch went well. Issuing the list again repeats the launches
    (engine/launch_memo.py does, for the next layer)."""

    def __enter__(self):
        global _recording
        self._outer = _recording
        self.calls: list = []
        _recording = self.calls
        return self

    def __exit__(self, *exc):
        global _recording
        _recording = self._outer
        return False


_pinned_stream: Optional[int] = None


def _stream() -> int:
    return _pinned_stream if _pinned_stream is not None else torch.cuda.current_stream().cuda_stream


@contextlib.contextmanager
def pinned_stream():
    """Inside the block every launch goes to the stream that is current on entry: one lookup for a whole forward
    pass instead of one per launch (the lookup costs more than the launch)."""
    global _pinned_stream
    previous = _pinned_stream
    _pinned_stream = torch.cuda.current_stream().cuda_stream
    try:
        yield
    finally:
        _pinned_stream = previous


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


LAUNCHES = 0     # kernels of this package launched so far (bench.py reports the count of its timed region)


def _check(code: int, what: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        return
    if code == DL_ERR_UNSUPPORTED:
        raise Unsupported(f"{what}: the kernel refuses these sizes")
    raise EngineError(f"{what}: CUDA error {code}")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise Unsupported(f"dtype {dtype} has no kernels (float32 and bfloat16 do)")


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise InvalidArgument("kernels take CUDA tensors only; there is no CPU path")


def _rows_contiguous(t: torch.Tensor, what: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise InvalidArgument(f"{what} must be 2-D with unit stride along its rows")


# ---------------------------------------------------------------------------------------------

def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[i, :] = table[ids[i], :] * scale; out is the float32 residual stream [rows, width]."""
    _cuda(table, ids, out)
    rows, width = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or ids.dtype != torch.int32 or not table.is_contiguous():
        raise InvalidArgument("embed: out float32 contiguous, ids int32, table contiguous")
    if table.shape[1] != width or ids.numel() < rows:
        raise InvalidArgument("embed: shapes disagree")
    _check(_fn("embedding", "dl_embed")(dtype_code(table.dtype), _p(table), _p(ids), _p(out), rows, width,
                                         table.shape[0], scale, _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, delta: Optional[torch.Tensor] = None,
            delta_scale: float = 1.0, rows: Optional[torch.Tensor] = None, write_residual: bool = True) -> None:
    """out[r] = rmsnorm(x[src] + delta_scale * delta[src]) * weight, src = rows[r] or r.

    x: float32 [n, width] residual stream, updated in place with the sum when `delta` is given and
    `write_residual`; delta: [n, width] of either dtype, or [parts, n, width] partial sums that are
    added in order; weight: float32 [width]; out: [n_out, width]."""
    _cuda(x, weight, out, delta, rows)
    width = x.shape[1]
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise InvalidArgument("rmsnorm: x and weight float32, x and out contiguous")
    if out.shape[1] != width or weight.numel() != width:
        raise InvalidArgument("rmsnorm: widths disagree")
    n_rows = out.shape[0]
    if rows is not None:
        if rows.dtype != torch.int32 or rows.numel() < n_rows:
            raise InvalidArgument("rmsnorm: rows must be int32 with one entry per output row")
        write_residual = False
    elif x.shape[0] < n_rows:
        raise InvalidArgument("rmsnorm: fewer input rows than output rows")
    parts, part_stride = _delta_parts(delta, width, "rmsnorm")
    dd = dtype_code(delta.dtype) if delta is not None else dtype_code(out.dtype)
    check_limits("norm", rows=x.shape[0])
    ahead, ahead_bytes = _take_ahead()
    _check(_fn("norm", "dl_rmsnorm")(dtype_code(out.dtype), dd, _p(x), _p(delta), delta_scale, _p(weight), eps,
                                      _p(out), _p(rows), n_rows, width, 1 if write_residual else 0, parts, part_stride,
                                      ahead, ahead_bytes, _stream()), "rmsnorm")


def _delta_parts(delta: Optional[torch.Tensor], width: int, what: str):
    """(number of partial sums, elements between them) of a delta that is [n, width] or [parts, n, width]."""
    if delta is None:
        return 1, 0
    if not delta.is_contiguous() or delta.shape[-1] != width or delta.dim() not in (2, 3):
        raise InvalidArgument(f"{what}: delta must be contiguous [n, width] or [parts, n, width]")
    if delta.dim() == 3:
        return delta.shape[0], delta.stride(0)
    return 1, 0


def residual_add(x: torch.Tensor, delta: torch.Tensor, scale: float = 1.0) -> None:
    """x += scale * delta over delta's rows (x float32); delta may be [parts, n, width] partial sums."""
    _cuda(x, delta)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise InvalidArgument("residual_add: x float32 and contiguous")
    parts, part_stride = _delta_parts(delta, x.shape[1], "residual_add")
    _check(_fn("norm", "dl_residual_add")(dtype_code(delta.dtype), _p(x), _p(delta), scale, delta.numel() // parts,
                                           parts, part_stride, _stream()), "residual_add")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = silu(gate_up[t, j]) * gate_up[t, inner + j]."""
    _cuda(gate_up, out)
    rows, inner = out.shape
    if gate_up.shape != (rows, 2 * inner) or not gate_up.is_contiguous() or not out.is_contiguous() \
            or gate_up.dtype != out.dtype:
        raise InvalidArgument("silu_mul: gate_up [rows, 2*inner] and out [rows, inner], contiguous, one dtype")
    _check(_fn("activation", "dl_silu_mul")(dtype_code(out.dtype), _p(gate_up), _p(out), rows, inner, _stream()),
           "silu_mul")


def rmsnorm_pair(x: torch.Tensor, weight_a: torch.Tensor, out_a: torch.Tensor, weight_b: Optional[torch.Tensor],
                 out_b: Optional[torch.Tensor], eps: float, delta_a: Optional[torch.Tensor] = None,
                 delta_b: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """Two norms of one row with one statistic: v = x[src] + (delta_a[src] + delta_b[src]); out_a[r] = rmsnorm(v) *
    weight_a, out_b[r] = rmsnorm(v) * weight_b (weight_b and out_b may both be None); src = rows[r] or r.

    x: float32 [n, width], updated in place with the sum unless `rows` picks a subset; each delta: [n, width] of either
    dtype or [parts, n, width] partial sums added in order, the two independently."""
    _cuda(x, weight_a, out_a, weight_b, out_b, delta_a, delta_b, rows)
    width = x.shape[1]
    if x.dtype != torch.float32 or weight_a.dtype != torch.float32 or not x.is_contiguous() or not out_a.is_contiguous() \
            or out_a.shape[1] != width or weight_a.numel() != width:
        raise InvalidArgument("rmsnorm_pair: x and weights float32, x and outputs contiguous, widths equal")
    if (out_b is None) != (weight_b is None) or (out_b is not None and (
            out_b.shape != out_a.shape or out_b.dtype != out_a.dtype or not out_b.is_contiguous()
            or weight_b.dtype != torch.float32 or weight_b.numel() != width)):
        raise InvalidArgument("rmsnorm_pair: the second output and weight come together and match the first")
    n_rows = out_a.shape[0]
    if rows is not None:
        if rows.dtype != torch.int32 or rows.numel() < n_rows:
            raise InvalidArgument("rmsnorm_pair: rows must be int32 with one entry per output row")
    elif x.shape[0] < n_rows:
        raise InvalidArgument("rmsnorm_pair: fewer input rows than output rows")
    parts_a, stride_a = _delta_parts(delta_a, width, "rmsnorm_pair")
    parts_b, stride_b = _delta_parts(delta_b, width, "rmsnorm_pair")
    check_limits("norm", rows=x.shape[0])
    _take_ahead()
    _check(_fn("norm", "dl_rmsnorm_pair")(
        dtype_code(out_a.dtype), _p(x), _p(delta_a), dtype_code(delta_a.dtype) if delta_a is not None else 0, parts_a,
        stride_a, _p(delta_b), dtype_code(delta_b.dtype) if delta_b is not None else 0, parts_b, stride_b, _p(weight_a),
        _p(weight_b), eps, _p(out_a), _p(out_b), _p(rows), n_rows, width, 0 if rows is not None else 1, _stream()),
        "rmsnorm_pair")


def relu2(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = max(x, 0)^2 elementwise (out may be x); both contiguous, of one dtype."""
    _cuda(x, out)
    if x.shape != out.shape or x.dtype != out.dtype or not x.is_contiguous() or not out.is_contiguous():
        raise InvalidArgument("relu2: x and out contiguous, of one shape and dtype")
    _check(_fn("activation", "dl_relu2")(dtype_code(x.dtype), _p(x), _p(out), x.numel(), _stream()), "relu2")


def gelu_tanh(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) elementwise (out may be x); both contiguous, of one dtype."""
    _cuda(x, out)
    if x.shape != out.shape or x.dtype != out.dtype or not x.is_contiguous() or not out.is_contiguous():
        raise InvalidArgument("gelu_tanh: x and out contiguous, of one shape and dtype")
    _check(_fn("activation", "dl_gelu_tanh")(dtype_code(x.dtype), _p(x), _p(out), x.numel(), _stream()), "gelu_tanh")


def norm_after_sum(x: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float, alpha: float = 1.0,
                   delta_scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> None:
    """x <- rmsnorm(alpha * x + delta_scale * delta) * weight, row by row, and out <- the same rows in out's dtype.

    x: float32 [n, width], replaced; delta: [n, width] of either dtype or [parts, n, width] partial sums added in
    order; delta_scale: float32 [width] or None; weight: float32 [width]; out: [n, width] or None. See
    csrc/norm_after_sum.cu."""
    _cuda(x, delta, weight, delta_scale, out)
    rows, width = x.shape
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or not x.is_contiguous() or weight.numel() != width:
        raise InvalidArgument("norm_after_sum: x and weight float32, x contiguous, widths equal")
    if delta_scale is not None and (delta_scale.dtype != torch.float32 or delta_scale.numel() != width):
        raise InvalidArgument("norm_after_sum: the scale of delta must be float32 [width]")
    if out is not None and (out.shape != x.shape or not out.is_contiguous()):
        raise InvalidArgument("norm_after_sum: out must be contiguous and of x's shape")
    parts, part_stride = _delta_parts(delta, width, "norm_after_sum")
    if delta.shape[-2] < rows:
        raise InvalidArgument("norm_after_sum: delta has fewer rows than x")
    od = dtype_code(out.dtype) if out is not None else dtype_code(delta.dtype)
    _take_ahead()
    _check(_fn("norm_after_sum", "dl_norm_after_sum")(
        od, dtype_code(delta.dtype), _p(x), _p(delta), parts, part_stride, _p(delta_scale), alpha, _p(weight), eps,
        _p(out), rows, width, _stream()), "norm_after_sum")


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (float32) in out's dtype; both contiguous and of one shape."""
    _cuda(x, out)
    if x.dtype != torch.float32 or x.shape != out.shape or not x.is_contiguous() or not out.is_contiguous():
        raise InvalidArgument("cast_rows: x float32, x and out contiguous and of one shape")
    _check(_fn("norm_after_sum", "dl_cast_rows")(dtype_code(out.dtype), _p(x), _p(out), x.numel(), _stream()), "cast_rows")


def ssm_conv(proj: torch.Tensor, col0: int, channels: int, taps_t: torch.Tensor, bias: Optional[torch.Tensor],
             state: torch.Tensor, keep_off: int, positions: torch.Tensor, row_request: torch.Tensor,
             row_slot: torch.Tensor, pos_start: torch.Tensor, out: torch.Tensor) -> None:
    """out[row, ch] = silu(bias[ch] + sum_k taps_t[k, ch] * u(position - (K - 1 - k), ch)), u = columns col0 .. col0 +
    channels of proj (the last tap is the current token's); inputs in front of a request's first row of the step come
    from its kept inputs, state[slot, keep_off + j * channels + ch] (oldest first). taps_t: float32 [K, channels],
    tap by tap; state: float32 [slots, n]. See csrc/ssm.cu."""
    taps = taps_t
    _cuda(proj, taps, bias, state, positions, row_request, row_slot, pos_start, out)
    _rows_contiguous(proj, "proj")
    rows = proj.shape[0]
    K = taps.shape[0]
    if taps.dtype != torch.float32 or not taps.is_contiguous() or taps.dim() != 2 or taps.shape[1] != channels \
            or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != channels)):
        raise InvalidArgument("ssm_conv: taps float32 [K, channels] and bias float32 [channels]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or keep_off + (K - 1) * channels > state.shape[1]:
        raise InvalidArgument("ssm_conv: state float32 [slots, n] with room for the kept inputs")
    if out.dtype != proj.dtype or out.shape != (rows, channels) or not out.is_contiguous() or col0 + channels > proj.shape[1]:
        raise InvalidArgument("ssm_conv: out contiguous [rows, channels] of proj's dtype; the channels lie inside proj")
    check_limits("ssm", requests=state.shape[0], rows=rows)
    _check(_fn("ssm", "dl_ssm_conv")(dtype_code(proj.dtype), _p(proj), proj.stride(0), col0, channels, _p(taps), _p(bias), K,
                                      _p(state), state.stride(0), keep_off, _p(positions), _p(row_request), _p(row_slot),
                                      _p(pos_start), _p(out), rows, _stream()), "ssm_conv")


def ssm_conv_keep(proj: torch.Tensor, col0: int, channels: int, K: int, state: torch.Tensor, keep_off: int,
                  q_start: torch.Tensor, state_slots: torch.Tensor, requests: int) -> None:
    """After a step's convolution: every request's last K - 1 inputs into its kept inputs (those it brought in this
    step, and the newest of the old ones where it brought fewer)."""
    _cuda(proj, state, q_start, state_slots)
    _rows_contiguous(proj, "proj")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or keep_off + (K - 1) * channels > state.shape[1]:
        raise InvalidArgument("ssm_conv_keep: state float32 [slots, n] with room for the kept inputs")
    check_limits("ssm", requests=state.shape[0], rows=proj.shape[0])
    _check(_fn("ssm", "dl_ssm_conv_keep")(dtype_code(proj.dtype), _p(proj), proj.stride(0), col0, channels, K, _p(state),
                                           state.stride(0), keep_off, _p(q_start), _p(state_slots), requests, _stream()),
           "ssm_conv_keep")


SSM_SEGMENT = 128      # tokens to a segment of a long portion, and the most a request brings to run as one piece


class SsmSegmentPlan:
    """The step plan of the state-space recurrence: the requests that bring more than SSM_SEGMENT tokens, cut into
    segments of at most that many, so that the segments of a portion run side by side (csrc/ssm.cu). int32 rows of 4:
    first a table of the long requests (first segment, segments, slot, 0), a third of the section's rows; behind it
    the segments (slot, first row of the step, rows, 0), request by request and in order. A step of T tokens has at
    most T // (SSM_SEGMENT + 1) long requests and T // SSM_SEGMENT segments more than that. `fill` returns (segments,
    long requests, rows of the table)."""

    name = "ssm_segments"

    def ints(self, max_tokens: int, max_requests: int) -> int:
        table = max(1, max_tokens // (SSM_SEGMENT + 1))
        return 4 * (2 * table + max_tokens // SSM_SEGMENT)

    @staticmethod
    def table_rows(section_ints: int) -> int:
        """Rows of the long requests' table in a section of that many integers: max_tokens // SSM_SEGMENT is the
        table's rows or one more, so the table is a third of the section, rounded down."""
        return max(1, section_ints // 12)

    def fill(self, host, shape):
        table = self.table_rows(len(host))
        longs, segs = [], []
        for n, r0, slot in zip(shape.q_len, shape.q_start, shape.slots):
            if n <= SSM_SEGMENT:
                continue
            first = len(segs)
            for t0 in range(0, n, SSM_SEGMENT):
                segs.append((slot, r0 + t0, min(SSM_SEGMENT, n - t0), 0))
            longs.append((first, len(segs) - first, slot, 0))
        if len(longs) > table or 4 * (table + len(segs)) > len(host):
            raise InvalidArgument("more long portions in a step than the step's buffers were made for")
        flat = [v for t in longs for v in t]
        host[:len(flat)] = flat
        flat = [v for t in segs for v in t]
        host[4 * table:4 * table + len(flat)] = flat
        return len(segs), len(longs), table

    @staticmethod
    def most_segments(max_tokens: int) -> int:
        return max_tokens // SSM_SEGMENT + max(1, max_tokens // (SSM_SEGMENT + 1))


SSM_SEGMENTS = SsmSegmentPlan()


def ssm_scan(u: torch.Tensor, proj: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
             d_skip: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, state_slots: torch.Tensor, y: torch.Tensor,
             requests: int, heads: int, head_dim: int, n_state: int, groups: int, planned=None,
             scratch: Optional[torch.Tensor] = None, seg_decay: Optional[torch.Tensor] = None) -> None:
    """The recurrence of every head over every request's rows of the step, from and into state[slot, :H*N*P] ([H, N,
    P]). u: [rows, H*P + 2*G*N] after the convolution (x | B | C); proj[row, dt_col + h]: the raw step size; y:
    float32 [rows, H*P]. `planned` = (the SsmSegmentPlan's integers on the device, what its fill returned): requests
    that bring more than SSM_SEGMENT tokens run as segments side by side, through `scratch` (float32, [segments, H*N*P]
    at least) and `seg_decay` (float32, [segments, H]); without it every request must bring at most SSM_SEGMENT tokens
    or runs as one piece however long it is. See csrc/ssm.cu."""
    _cuda(u, proj, dt_bias, a_log, d_skip, state, q_start, state_slots, y, scratch, seg_decay)
    _rows_contiguous(u, "u")
    _rows_contiguous(proj, "proj")
    inner = heads * head_dim
    if u.dtype != proj.dtype or u.shape[1] != inner + 2 * groups * n_state or dt_col + heads > proj.shape[1]:
        raise InvalidArgument("ssm_scan: u is [rows, H*P + 2*G*N] of proj's dtype and proj holds H step sizes from dt_col")
    if any(t.dtype != torch.float32 or t.numel() != heads for t in (dt_bias, a_log, d_skip)):
        raise InvalidArgument("ssm_scan: dt_bias, a_log and d are float32 [heads]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < inner * n_state:
        raise InvalidArgument("ssm_scan: state float32 [slots, >= H*N*P]")
    if y.dtype != torch.float32 or not y.is_contiguous() or y.shape != (u.shape[0], inner):
        raise InvalidArgument("ssm_scan: y float32 contiguous [rows, H*P]")
    whole_up_to, segs, n_segs, longs, n_long = 1 << 30, None, 0, None, 0
    if planned is not None:
        ints, (n_segs, n_long, long_cap) = planned
        if n_segs:
            if scratch is None or seg_decay is None or scratch.dtype != torch.float32 or seg_decay.dtype != torch.float32 \
                    or scratch.numel() < n_segs * inner * n_state or seg_decay.numel() < n_segs * heads:
                raise InvalidArgument("ssm_scan: scratch float32 [segments, H*N*P] and seg_decay float32 [segments, H]")
            longs, segs = ints, ints[4 * long_cap:]
        whole_up_to = SSM_SEGMENT
    check_limits("ssm", requests=state.shape[0], rows=u.shape[0])
    _check(_fn("ssm", "dl_ssm_scan")(dtype_code(u.dtype), _p(u), u.stride(0), _p(proj), proj.stride(0), dt_col, _p(dt_bias),
                                      _p(a_log), _p(d_skip), _p(state), state.stride(0), _p(q_start), _p(state_slots),
                                      _p(y), requests, heads, head_dim, n_state, groups, whole_up_to, _p(segs), n_segs,
                                      _p(longs), n_long, _p(scratch), _p(seg_decay), _stream()), "ssm_scan")


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float, parts: int,
                     out: torch.Tensor) -> None:
    """out = norm_parts(y * silu(z)) * weight: each of `parts` equal pieces of a row by its own root mean square. y:
    float32 [rows, inner]; z: rows whose first `inner` columns are the gate; out: [rows, inner] of z's dtype."""
    _cuda(y, z, weight, out)
    _rows_contiguous(z, "z")
    rows, inner = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous() or z.shape[1] < inner or weight.dtype != torch.float32 \
            or weight.numel() != inner or out.shape != y.shape or out.dtype != z.dtype or not out.is_contiguous():
        raise InvalidArgument("gated_group_norm: y float32 [rows, inner], z at least as wide, weight float32 [inner], out like y in z's dtype")
    if parts <= 0 or inner % parts:
        raise InvalidArgument(f"gated_group_norm: {inner} channels do not divide into {parts} parts")
    _check(_fn("ssm", "dl_gated_group_norm")(dtype_code(z.dtype), _p(y), _p(z), z.stride(0), _p(weight), eps, _p(out),
                                              rows, inner, parts, _stream()), "gated_group_norm")


def latent_prep(proj: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, rot: int, q_weight: torch.Tensor,
                kv_weight: torch.Tensor, eps: float, freq: Optional[torch.Tensor], positions: torch.Tensor,
                row_slot: torch.Tensor, block_table: torch.Tensor, cache: torch.Tensor, page_size: int,
                cq: torch.Tensor) -> None:
    """Per row of proj = [query latent | latent | key part | ...]: cq = rmsnorm(query latent) * q_weight, and the row's
    record [rmsnorm(latent) * kv_weight | key part with its first `rot` numbers turned by the position] into the paged
    cache [pages, page_size, kv_rank + rot_dim]. freq: float64 [rot / 2]. See csrc/latent_attention.cu."""
    _cuda(proj, q_weight, kv_weight, freq, positions, row_slot, block_table, cache, cq)
    _rows_contiguous(proj, "proj")
    rows = proj.shape[0]
    if proj.shape[1] < q_rank + kv_rank + rot_dim:
        raise InvalidArgument("latent_prep: proj is narrower than its three pieces")
    if q_weight.dtype != torch.float32 or q_weight.numel() != q_rank or kv_weight.dtype != torch.float32 or kv_weight.numel() != kv_rank:
        raise InvalidArgument("latent_prep: norm weights float32 [q_rank] and [kv_rank]")
    if rot and (freq is None or freq.dtype != torch.float64 or freq.numel() != rot // 2):
        raise InvalidArgument("latent_prep: freq float64 [rot / 2]")
    if cache.dtype != proj.dtype or not cache.is_contiguous() or cache.dim() != 3 or cache.shape[1] != page_size \
            or cache.shape[2] != kv_rank + rot_dim:
        raise InvalidArgument("latent_prep: the cache must be contiguous [pages, page_size, kv_rank + rot_dim] of proj's dtype")
    if cq.dtype != proj.dtype or cq.shape != (rows, q_rank) or not cq.is_contiguous():
        raise InvalidArgument("latent_prep: cq contiguous [rows, q_rank] of proj's dtype")
    if block_table.dtype != torch.int32 or block_table.stride(-1) != 1:
        raise InvalidArgument("latent_prep: block_table must be int32 rows")
    check_limits("latent_attention", pages=cache.shape[0], requests=block_table.shape[0], rows=rows)
    _check(_fn("latent_attention", "dl_latent_prep")(
        dtype_code(proj.dtype), _p(proj), proj.stride(0), q_rank, kv_rank, rot_dim, rot, _p(q_weight), _p(kv_weight), eps,
        _p(freq), _p(positions), _p(row_slot), _p(block_table), block_table.stride(0), page_size, _p(cq), _p(cache), rows,
        _stream()), "latent_prep")


def rotate_pairs(q: torch.Tensor, head_in: int, in_off: int, out: torch.Tensor, head_out: int, out_off: int, r: int,
                 rot: int, freq: Optional[torch.Tensor], positions: torch.Tensor, heads: int) -> None:
    """out[row, h * head_out + out_off + i] = q[row, h * head_in + in_off + i] for i < r, the first `rot` of them
    turned in interleaved pairs (2i, 2i + 1) by position * freq[i]."""
    _cuda(q, out, freq, positions)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if q.dtype != out.dtype or q.shape[0] != out.shape[0] or (heads - 1) * head_in + in_off + r > q.shape[1] \
            or (heads - 1) * head_out + out_off + r > out.shape[1]:
        raise InvalidArgument("rotate_pairs: q and out of one dtype and row count, the heads' pieces inside them")
    if rot and (freq is None or freq.dtype != torch.float64 or freq.numel() != rot // 2):
        raise InvalidArgument("rotate_pairs: freq float64 [rot / 2]")
    _check(_fn("latent_attention", "dl_rotate_pairs")(
        dtype_code(q.dtype), _p(q), q.stride(0), head_in, in_off, _p(out), out.stride(0), head_out, out_off, r, rot,
        _p(freq), _p(positions), q.shape[0], heads, _stream()), "rotate_pairs")


def head_linear(x: torch.Tensor, head_in: int, n_in: int, w: torch.Tensor, out: torch.Tensor, head_out: int,
                gate: Optional[torch.Tensor] = None, gate_head: int = 0) -> None:
    """out[row, h * head_out + j] = sum_i x[row, h * head_in + i] * w[h, i, j] for every head h (a block-diagonal
    product), times sigmoid(gate[row, h * gate_head + j]) when a gate is given. w: contiguous [H, n_in, n_out]."""
    _cuda(x, w, out, gate)
    _rows_contiguous(x, "x")
    _rows_contiguous(out, "out")
    if w.dim() != 3 or not w.is_contiguous() or w.shape[1] != n_in or w.dtype != x.dtype or out.dtype != x.dtype:
        raise InvalidArgument("head_linear: w contiguous [H, n_in, n_out]; x, w and out of one dtype")
    H, n_out = w.shape[0], w.shape[2]
    if (H - 1) * head_in + n_in > x.shape[1] or (H - 1) * head_out + n_out > out.shape[1] or out.shape[0] != x.shape[0]:
        raise InvalidArgument("head_linear: the heads' pieces do not fit x or out")
    if gate is not None:
        _rows_contiguous(gate, "gate")
        if gate.dtype != x.dtype or gate.shape[0] < x.shape[0] or (H - 1) * gate_head + n_out > gate.shape[1]:
            raise InvalidArgument("head_linear: the gate's pieces do not fit")
    gate_stride = gate.stride(0) if gate is not None else 0
    if (x.dtype == torch.bfloat16 and n_in % 8 == 0 and n_out % 8 == 0 and x.stride(0) % 8 == 0 and head_in % 8 == 0
            and out.stride(0) % 2 == 0 and head_out % 2 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and out.data_ptr() % 4 == 0):
        # the tensor-core kernel (csrc/head_linear_tc.cu)
        _check(_fn("head_linear_tc", "dl_head_linear_tc")(
            _p(x), x.stride(0), head_in, n_in, _p(w), n_out, _p(out), out.stride(0), head_out, _p(gate), gate_stride,
            gate_head, x.shape[0], H, _stream()), "head_linear")
        return
    _check(_fn("latent_attention", "dl_head_linear")(
        dtype_code(x.dtype), _p(x), x.stride(0), head_in, n_in, _p(w), n_out, _p(out), out.stride(0), head_out, _p(gate),
        gate_stride, gate_head, x.shape[0], H, _stream()), "head_linear")


def latent_attention(qw: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, positions: torch.Tensor,
                     row_slot: torch.Tensor, sink: Optional[torch.Tensor], out: torch.Tensor, heads: int, kv_rank: int,
                     rot_dim: int, page_size: int, scale: float, window: int) -> None:
    """Every row's wide queries [H, kv_rank + rot_dim] over the records of its request's window; out [rows, H,
    kv_rank] = softmax-weighted sum of the records' latents, the denominator also holding exp(sink[h]) when sinks are
    given. The plain kernel; see csrc/latent_attention.cu."""
    _cuda(qw, cache, block_table, positions, row_slot, sink, out)
    _rows_contiguous(qw, "qw")
    _rows_contiguous(out, "out")
    rw = kv_rank + rot_dim
    if qw.dtype != cache.dtype or out.dtype != qw.dtype or qw.shape[1] < heads * rw or out.shape[1] < heads * kv_rank:
        raise InvalidArgument("latent_attention: qw, cache and out of one dtype; qw [rows, H*(R+r)], out [rows, H*R]")
    if cache.dim() != 3 or cache.shape[1] != page_size or cache.shape[2] != rw or not cache.is_contiguous():
        raise InvalidArgument("latent_attention: the cache is not contiguous [pages, page_size, kv_rank + rot_dim]")
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != heads):
        raise InvalidArgument("latent_attention: sinks float32 [heads]")
    check_limits("latent_attention", pages=cache.shape[0], requests=block_table.shape[0], rows=qw.shape[0])
    _check(_fn("latent_attention", "dl_latent_attention")(
        dtype_code(qw.dtype), _p(qw), qw.stride(0), _p(cache), _p(block_table), block_table.stride(0), _p(positions),
        _p(row_slot), _p(sink), _p(out), out.stride(0), qw.shape[0], heads, kv_rank, rot_dim, page_size, scale, window,
        _stream()), "latent_attention")


# Records of the tensor-core latent attention by one bulk copy each (completion on an mbarrier) instead of 16-byte
# cp.async pieces; DYNALM_LATENT_BULK=0 keeps the pieces.
LATENT_BULK = os.environ.get("DYNALM_LATENT_BULK", "1") != "0"


def latent_flash_fits(kv_rank: int, rot_dim: int) -> bool:
    """Whether the tensor-core latent attention's shared memory (32 query units and two tiles of 64 records) fits a block."""
    stride = ((kv_rank + rot_dim + 15) & ~15) + 8
    return 2 * ((32 + 128) * stride + 32 * 72) + 4 * 256 <= 220 * 1024


def latent_attention_flash(qw: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, tiles: torch.Tensor,
                           n_tiles: int, sink: Optional[torch.Tensor], out: torch.Tensor, heads: int, kv_rank: int,
                           rot_dim: int, page_size: int, scale: float, window: int, heads_per_block: int, parts: int = 1,
                           scratch: Optional[torch.Tensor] = None) -> None:
    """latent_attention on bf16 tensor cores: one block per (query tile, group of `heads_per_block` heads), the tiles
    int32 [n_tiles, 4] = (request slot, first row, rows, first position) with at most 32 // heads_per_block rows each.
    parts > 1: the key tiles of every query tile are dealt over that many blocks, which leave their shares in `scratch`
    (float32, rows * heads * parts * (kv_rank + 2) at least) for a merge kernel: for steps of few rows, which would
    leave most of the GPU idle. See csrc/latent_attention_flash.cu."""
    _cuda(qw, cache, block_table, tiles, sink, out)
    _rows_contiguous(qw, "qw")
    _rows_contiguous(out, "out")
    rw = kv_rank + rot_dim
    if any(t.dtype != torch.bfloat16 for t in (qw, cache, out)):
        raise Unsupported("latent_attention_flash: bfloat16 only")
    if qw.shape[1] < heads * rw or out.shape[1] < heads * kv_rank or cache.dim() != 3 or cache.shape[1] != page_size \
            or cache.shape[2] != rw or not cache.is_contiguous():
        raise InvalidArgument("latent_attention_flash: qw [rows, H*(R+r)], out [rows, H*R], cache contiguous [pages, page_size, R+r]")
    if tiles.dtype != torch.int32 or tiles.numel() < 4 * n_tiles:
        raise InvalidArgument("latent_attention_flash: tiles int32 [n_tiles, 4]")
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != heads):
        raise InvalidArgument("latent_attention_flash: sinks float32 [heads]")
    rows = qw.shape[0]
    if parts > 1 and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < rows * heads * parts * (kv_rank + 2)):
        raise InvalidArgument("latent_attention_flash: scratch float32 [rows, heads, parts, kv_rank + 2]")
    check_limits("latent_attention_flash", pages=cache.shape[0], requests=block_table.shape[0], rows=rows)
    _take_ahead()
    _check(_fn("latent_attention_flash", "dl_latent_attention_flash")(
        _p(qw), qw.stride(0), _p(cache), _p(block_table), block_table.stride(0), _p(tiles), n_tiles, _p(sink), _p(out),
        out.stride(0), heads, kv_rank, rot_dim, page_size, scale, window, heads_per_block, parts,
        _p(scratch) if parts > 1 else None, rows, 1 if LATENT_BULK else 0, _p(_status_word(qw.device)), _stream()),
        "latent_attention_flash")
    if parts > 1:
        global LAUNCHES
        LAUNCHES += 1


def qk_norm_cache_write(qkv: torch.Tensor, positions: torch.Tensor, row_slot: torch.Tensor,
                        block_table: Optional[torch.Tensor], cache: Optional[torch.Tensor], k_off: int, v_off: int,
                        q_weight: torch.Tensor, k_weight: Optional[torch.Tensor], eps: float, temp_coef: float,
                        temp_every: int, n_q_units: int, n_k_units: int, dim: int, v_width: int, page_size: int,
                        write_cache: bool = True) -> None:
    """Per-unit RMS norm of the queries of `qkv` in place (with the position-dependent temperature when temp_every >
    0), and, with write_cache, the normalised keys and the values into each row's record of the paged cache
    [pages, page_size, record]; see csrc/qk_norm_cache.cu. qkv: [rows, >= (n_q_units + n_k_units) * dim + v_width]."""
    _cuda(qkv, positions, row_slot, block_table, cache, q_weight, k_weight)
    _rows_contiguous(qkv, "qkv")
    rows = qkv.shape[0]
    need = n_q_units * dim + ((n_k_units * dim + v_width) if write_cache else 0)
    if qkv.shape[1] < need:
        raise InvalidArgument("qk_norm_cache_write: qkv is narrower than its units")
    if q_weight.dtype != torch.float32 or q_weight.numel() != dim:
        raise InvalidArgument("qk_norm_cache_write: the query norm weight must be float32 [dim]")
    record = 0
    if write_cache:
        if cache is None or block_table is None or k_weight is None:
            raise InvalidArgument("qk_norm_cache_write: a cache write needs the cache, a block table and the key norm weight")
        if cache.dtype != qkv.dtype or not cache.is_contiguous() or cache.dim() != 3 or cache.shape[1] != page_size:
            raise InvalidArgument("qk_norm_cache_write: the cache must be contiguous [pages, page_size, record] of qkv's dtype")
        record = cache.shape[2]
        if k_off < 0 or v_off < 0 or k_off + n_k_units * dim > record or v_off + v_width > record:
            raise InvalidArgument("qk_norm_cache_write: keys or values do not fit the record")
        if k_weight.dtype != torch.float32 or k_weight.numel() != dim:
            raise InvalidArgument("qk_norm_cache_write: the key norm weight must be float32 [dim]")
        if block_table.dtype != torch.int32 or block_table.stride(-1) != 1:
            raise InvalidArgument("qk_norm_cache_write: block_table must be int32 rows")
        check_limits("qk_norm_cache", pages=cache.shape[0], requests=block_table.shape[0], rows=rows)
    max_blocks = block_table.stride(0) if block_table is not None else 0
    _check(_fn("qk_norm_cache", "dl_qk_norm_cache_write")(
        dtype_code(qkv.dtype), _p(qkv), qkv.stride(0), _p(positions), _p(row_slot), _p(block_table), max_blocks,
        _p(cache), record, k_off, v_off, _p(q_weight), _p(k_weight), eps, temp_coef, int(temp_every), rows, n_q_units,
        n_k_units, dim, v_width, page_size, 1 if write_cache else 0, _stream()), "qk_norm_cache_write")


def diff_attention(q: torch.Tensor, cache: torch.Tensor, k_off: int, v_off: int, block_table: torch.Tensor,
                   positions: torch.Tensor, row_slot: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                   dim: int, vdim: int, page_size: int, scale: float, softcap: float, lam: torch.Tensor,
                   out_scale: float, eps: float) -> None:
    """Differential attention of every row over its request's cached records, the plain kernel; see
    csrc/attention_diff.cu. q: [rows, >= n_heads * 2 * dim]; out: [rows, >= n_heads * vdim]; cache: [pages, page_size,
    record]; lam: one float32 on the device."""
    _cuda(q, cache, block_table, positions, row_slot, out, lam)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if dim > 256 or vdim > 256 or n_heads % n_kv_heads:
        raise Unsupported(f"diff attention: dim {dim} / vdim {vdim} (at most 256), heads {n_heads}:{n_kv_heads}")
    if q.dtype != out.dtype or cache.dtype != q.dtype or lam.dtype != torch.float32:
        raise InvalidArgument("diff attention: q, out and the cache share one dtype; lambda is float32")
    if cache.dim() != 3 or cache.shape[1] != page_size or not cache.is_contiguous() \
            or k_off + n_kv_heads * 2 * dim > cache.shape[2] or v_off + n_kv_heads * vdim > cache.shape[2]:
        raise InvalidArgument("diff attention: the cache is not [pages, page_size, record] with room for keys and values")
    check_limits("attention_diff", pages=cache.shape[0], requests=block_table.shape[0], rows=q.shape[0])
    _check(_fn("attention_diff", "dl_diff_attention")(
        dtype_code(q.dtype), _p(q), q.stride(0), _p(cache), cache.shape[2], k_off, v_off, _p(block_table),
        block_table.stride(0), _p(positions), _p(row_slot), _p(out), out.stride(0), q.shape[0], n_heads, n_kv_heads, dim,
        vdim, page_size, scale, softcap, _p(lam), out_scale, eps, _stream()), "diff_attention")


def _diff_fast_checks(q, cache, out, block_table, lam, k_off, v_off, n_heads, n_kv_heads, dim, vdim, page_size, what):
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if any(t.dtype != torch.bfloat16 for t in (q, cache, out)) or lam.dtype != torch.float32:
        raise Unsupported(f"{what}: bfloat16 only (lambda float32)")
    if dim % 16 or vdim % 16 or dim > 128 or vdim > 128 or n_heads % n_kv_heads or page_size & (page_size - 1):
        raise Unsupported(f"{what}: dim {dim} and vdim {vdim} (multiples of 16 up to 128), heads {n_heads}:{n_kv_heads}, "
                          f"page size {page_size} (a power of two)")
    if cache.dim() != 3 or cache.shape[1] != page_size or not cache.is_contiguous() \
            or k_off + n_kv_heads * 2 * dim > cache.shape[2] or v_off + n_kv_heads * vdim > cache.shape[2]:
        raise InvalidArgument(f"{what}: the cache is not [pages, page_size, record] with room for keys and values")
    if q.stride(0) % 8 or out.stride(0) % 2 or q.data_ptr() % 16 or out.data_ptr() % 4 or cache.data_ptr() % 16 \
            or cache.shape[2] % 8 or k_off % 8 or v_off % 8:
        raise Unsupported(f"{what}: q rows and records must be 16-byte aligned, out rows 4-byte aligned")
    if block_table.dtype != torch.int32 or block_table.stride(-1) != 1:
        raise InvalidArgument(f"{what}: block_table must be int32 rows")


def diff_attention_prefill(q: torch.Tensor, cache: torch.Tensor, k_off: int, v_off: int, block_table: torch.Tensor,
                           q_tiles: torch.Tensor, n_tiles: int, out: torch.Tensor, n_heads: int, n_kv_heads: int, dim: int,
                           vdim: int, page_size: int, scale: float, softcap: float, lam: torch.Tensor, out_scale: float,
                           eps: float) -> None:
    """Differential flash attention of query tiles over paged records, bfloat16; see csrc/attention_diff_flash.cu.
    q_tiles: int32 [n_tiles, 4] = (request slot, first row, rows <= 128, first position)."""
    _cuda(q, cache, block_table, q_tiles, out, lam)
    _diff_fast_checks(q, cache, out, block_table, lam, k_off, v_off, n_heads, n_kv_heads, dim, vdim, page_size,
                      "diff attention (prompt)")
    if q_tiles.dtype != torch.int32 or q_tiles.numel() < 4 * n_tiles or q_tiles.data_ptr() % 16:
        raise InvalidArgument("diff attention (prompt): q_tiles must be int32 [n_tiles, 4], 16-byte aligned")
    check_limits("attention_diff_flash", pages=cache.shape[0], requests=block_table.shape[0], rows=q.shape[0])
    _check(_fn("attention_diff_flash", "dl_diff_attention_prefill")(
        _p(q), q.stride(0), _p(cache), cache.shape[2], k_off, v_off, _p(block_table), block_table.stride(0), _p(q_tiles),
        n_tiles, _p(out), out.stride(0), n_heads, n_kv_heads, dim, vdim, page_size, scale, softcap, _p(lam), out_scale, eps,
        _stream()), "diff_attention_prefill")


def diff_decode_scratch_floats(rows: int, n_heads: int, vdim: int, n_split: int) -> int:
    """Floats of scratch `diff_attention_decode` needs."""
    return 0 if n_split <= 1 else rows * n_heads * n_split * 2 * (vdim + 2)


def diff_attention_decode(q: torch.Tensor, cache: torch.Tensor, k_off: int, v_off: int, block_table: torch.Tensor,
                          positions: torch.Tensor, row_slot: torch.Tensor, out: torch.Tensor, scratch: Optional[torch.Tensor],
                          n_heads: int, n_kv_heads: int, dim: int, vdim: int, page_size: int, scale: float, softcap: float,
                          lam: torch.Tensor, out_scale: float, eps: float, n_split: int) -> None:
    """Differential split-KV attention for rows that bring one token each, bfloat16; see csrc/attention_diff_flash.cu.
    `scratch`: float32 with at least diff_decode_scratch_floats(...) elements when n_split > 1."""
    _cuda(q, cache, block_table, positions, row_slot, out, lam, scratch)
    _diff_fast_checks(q, cache, out, block_table, lam, k_off, v_off, n_heads, n_kv_heads, dim, vdim, page_size,
                      "diff attention (single tokens)")
    rows = q.shape[0]
    need = diff_decode_scratch_floats(rows, n_heads, vdim, n_split)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise InvalidArgument(f"diff attention (single tokens): scratch must be float32 with at least {need} elements")
    check_limits("attention_diff_flash", pages=cache.shape[0], requests=block_table.shape[0], rows=rows)
    _check(_fn("attention_diff_flash", "dl_diff_attention_decode")(
        _p(q), q.stride(0), _p(cache), cache.shape[2], k_off, v_off, _p(block_table), block_table.stride(0), _p(positions),
        _p(row_slot), _p(out), out.stride(0), _p(scratch), rows, n_heads, n_kv_heads, dim, vdim, page_size, scale, softcap,
        _p(lam), out_scale, eps, int(n_split), _stream()), "diff_attention_decode")
    if n_split > 1:
        global LAUNCHES
        LAUNCHES += 1          # the merge kernel


def rope_cache_write(qkv: torch.Tensor, positions: torch.Tensor, row_request: torch.Tensor,
                     block_table: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                     v_cache: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rotary_dim: int,
                     pos_scale: float, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int,
                     write_cache: bool = True) -> None:
    """Rotate the q heads of `qkv` in place; rotate the k heads and copy the v heads into the paged
    cache at each row's position. qkv: [rows, >= (n_heads + 2 n_kv_heads) head_dim]."""
    _cuda(qkv, positions, row_request, block_table, k_cache, v_cache, inv_freq)
    _rows_contiguous(qkv, "qkv")
    rows = qkv.shape[0]
    need = (n_heads + (2 * n_kv_heads if write_cache else 0)) * head_dim
    if qkv.shape[1] < need:
        raise InvalidArgument("rope_cache_write: qkv is narrower than its heads")
    if write_cache:
        if k_cache is None or v_cache is None or block_table is None:
            raise InvalidArgument("rope_cache_write: a cache write needs k_cache, v_cache and a block table")
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype or not k_cache.is_contiguous() or not v_cache.is_contiguous():
            raise InvalidArgument("rope_cache_write: cache arrays must be contiguous and of qkv's dtype")
        if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim):
            raise InvalidArgument("rope_cache_write: cache shape is not [pages, page_size, kv_heads, head_dim]")
        if block_table.dtype != torch.int32 or block_table.stride(-1) != 1:
            raise InvalidArgument("rope_cache_write: block_table must be int32 rows")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() * 2 != rotary_dim):
        raise InvalidArgument("rope_cache_write: inv_freq must be float32 [rotary_dim / 2]")
    if rotary_dim > head_dim or rotary_dim % 2:
        raise Unsupported(f"rotary_dim {rotary_dim} does not fit head_dim {head_dim}")
    max_blocks = block_table.stride(0) if block_table is not None else 0
    if write_cache:
        check_limits("rope_cache", pages=k_cache.shape[0], requests=block_table.shape[0], rows=rows)
    _check(_fn("rope_cache", "dl_rope_cache_write")(
        dtype_code(qkv.dtype), _p(qkv), qkv.stride(0), _p(positions), _p(row_request), _p(block_table), max_blocks,
        _p(k_cache), _p(v_cache), _p(inv_freq), rotary_dim if inv_freq is not None else 0, pos_scale, rows, n_heads,
        n_kv_heads, head_dim, page_size, 1 if write_cache else 0, _stream()), "rope_cache_write")


def paged_attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                            positions: torch.Tensor, row_request: torch.Tensor, out: torch.Tensor, n_heads: int,
                            n_kv_heads: int, head_dim: int, page_size: int, scale: float, window: int = 0) -> None:
    """Causal attention of every row over its request's cached keys; see csrc/attention_generic.cu.
    q, out: [rows, >= n_heads * head_dim] views with unit column stride."""
    _cuda(q, k_cache, v_cache, block_table, positions, row_request, out)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if head_dim % 16 or head_dim > 256:
        raise Unsupported(f"attention: head_dim {head_dim} must be a multiple of 16, at most 256")
    if n_heads % n_kv_heads:
        raise Unsupported(f"attention: {n_heads} heads do not divide into {n_kv_heads} KV heads")
    if q.dtype != out.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise InvalidArgument("attention: q, out and the cache must share one dtype")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise InvalidArgument("attention: cache shape is not [pages, page_size, kv_heads, head_dim]")
    check_limits("attention_generic", pages=k_cache.shape[0], requests=block_table.shape[0], rows=q.shape[0])
    _check(_fn("attention_generic", "dl_paged_attention_generic")(
        dtype_code(q.dtype), _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), block_table.stride(0),
        _p(positions), _p(row_request), _p(out), out.stride(0), q.shape[0], n_heads, n_kv_heads, head_dim, page_size,
        scale, window, _stream()), "paged_attention_generic")


def decode_scratch_floats(rows: int, n_heads: int, head_dim: int, n_split: int) -> int:
    """Floats of scratch `paged_attention_decode` needs."""
    return 0 if n_split <= 1 else rows * n_heads * n_split * (head_dim + 2)


def paged_attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                           positions: torch.Tensor, row_request: torch.Tensor, out: torch.Tensor,
                           scratch: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, head_dim: int,
                           page_size: int, scale: float, window: int, n_split: int, tensor_cores: bool = False) -> None:
    """Split-KV attention for rows that bring few tokens; see csrc/attention_decode.cu. `scratch`:
    float32 with at least decode_scratch_floats(...) elements when n_split > 1. `tensor_cores`
    picks the mma variant (bfloat16, head_dim up to 128)."""
    _cuda(q, k_cache, v_cache, block_table, positions, row_request, out, scratch)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    rows = q.shape[0]
    if page_size & (page_size - 1):
        raise Unsupported(f"decode attention: page size {page_size} is not a power of two")
    if head_dim % 16 or head_dim > 256 or n_heads % n_kv_heads:
        raise Unsupported(f"decode attention: head_dim {head_dim} / heads {n_heads}:{n_kv_heads} not supported")
    if q.dtype != out.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise InvalidArgument("decode attention: q, out and the cache must share one dtype")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise InvalidArgument("decode attention: cache shape is not [pages, page_size, kv_heads, head_dim]")
    need = decode_scratch_floats(rows, n_heads, head_dim, n_split)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise InvalidArgument(f"decode attention: scratch must be float32 with at least {need} elements")
    check_limits("attention_decode", pages=k_cache.shape[0], requests=block_table.shape[0], rows=rows)
    if tensor_cores:
        if q.dtype != torch.bfloat16 or head_dim > 128 or q.stride(0) % 8 or q.data_ptr() % 16:
            raise Unsupported("decode attention (tensor cores): bfloat16, head_dim up to 128, 16-byte aligned q rows")
        ahead, ahead_bytes = _take_ahead()
        _check(_fn("attention_decode", "dl_paged_attention_decode_tc")(
            _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), block_table.stride(0), _p(positions),
            _p(row_request), _p(out), out.stride(0), _p(scratch), rows, n_heads, n_kv_heads, head_dim, page_size, scale,
            window, n_split, ahead, ahead_bytes, _stream()), "paged_attention_decode_tc")
        return
    _check(_fn("attention_decode", "dl_paged_attention_decode")(
        dtype_code(q.dtype), _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), block_table.stride(0),
        _p(positions), _p(row_request), _p(out), out.stride(0), _p(scratch), rows, n_heads, n_kv_heads, head_dim,
        page_size, scale, window, n_split, _stream()), "paged_attention_decode")


def decode_tile_keys(head_dim: int) -> int:
    """Keys per tile of the tensor-core decode attention (what its plans count keys in); the table of
    csrc/attention_decode.cu (dl_paged_attention_decode_tile), kept here so that a plan can be made without the
    library."""
    return 16 if head_dim >= 96 or head_dim == 64 else 32


def paged_attention_decode_planned(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                                   positions: torch.Tensor, row_request: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor,
                                   counters: torch.Tensor, plan: torch.Tensor, unit_cap: int, part_stride: int, n_heads: int,
                                   n_kv_heads: int, head_dim: int, page_size: int, scale: float, window: int) -> None:
    """The tensor-core split-KV attention with the keys of all rows dealt into units by the host (`plan`, see
    kernels/attention.DecodeUnits): one block per unit, `unit_cap` blocks launched; the last block of a row's group of
    heads to finish merges the row's parts. bfloat16, head_dim up to 128. scratch: float32, rows * n_heads * part_stride *
    (head_dim + 2) elements; counters: int32, rows * KV-head chunks, zero (the kernel leaves them zero)."""
    _cuda(q, k_cache, v_cache, block_table, positions, row_request, out, scratch, counters, plan)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    rows = q.shape[0]
    chunks = n_kv_heads * -(-(n_heads // n_kv_heads) // 16)
    if q.dtype != torch.bfloat16 or head_dim % 16 or head_dim > 128 or n_heads % n_kv_heads or page_size & (page_size - 1) \
            or q.stride(0) % 8 or q.data_ptr() % 16:
        raise Unsupported("decode attention (planned): bfloat16, head_dim up to 128, 16-byte aligned q rows")
    if q.dtype != out.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise InvalidArgument("decode attention: q, out and the cache must share one dtype")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise InvalidArgument("decode attention: cache shape is not [pages, page_size, kv_heads, head_dim]")
    if scratch.dtype != torch.float32 or scratch.numel() < rows * n_heads * part_stride * (head_dim + 2) \
            or counters.dtype != torch.int32 or counters.numel() < rows * chunks or plan.dtype != torch.int32 \
            or plan.numel() < 4 + 4 * unit_cap or plan.data_ptr() % 16:
        raise InvalidArgument("decode attention (planned): scratch, counters or plan too small or of the wrong type")
    check_limits("attention_decode", pages=k_cache.shape[0], requests=block_table.shape[0], rows=rows)
    ahead, ahead_bytes = _take_ahead()
    _check(_fn("attention_decode", "dl_paged_attention_decode_planned")(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), block_table.stride(0), _p(positions),
        _p(row_request), _p(out), out.stride(0), _p(scratch), rows, n_heads, n_kv_heads, head_dim, page_size, scale,
        window, _p(plan), _p(counters), unit_cap, part_stride, ahead, ahead_bytes, _stream()),
        "paged_attention_decode_planned")


QKV_ROPE_TCGEN05_HEAD_DIMS = (64, 128)
# From how many rounds of 256-wide tiles over the SMs the tcgen05 product with the rotating epilogue is ahead of the
# product followed by the rotation kernel. The rotating epilogue of a tile takes about 10 us more than the plain one
# and only hides behind the next tile of the same block. Measured in CUDA graphs (us: fused / own product + rotation /
# library product + rotation), head size 128, width 3072 with 24+8+8 heads: 544 rows 27.7 / 21.1 / 20.4, 1,024 rows
# 43.8 / 35.5 / 29.8, 2,048 rows (2.2 rounds) 63.1 / 58.1 / 55.0, 4,096 rows 103 / 112 / 102; width 4096 with 32+8+8
# heads: 1,024 rows 58.4 / 51.2 / 44.0, 2,048 rows (2.6 rounds) 90.1 / 94.7 / 85.4, 4,096 rows 169 / 191 / 188. At
# head size 64 (width 2048, 32+8+8 heads) the two are level from 544 rows on (15.6 / 15.4, 27.5 / 28.8 at 2,048 rows),
# and one launch less is worth more to a step that waits for the host.
QKV_ROPE_TCGEN05_MIN_ROUNDS = {64: 0.0, 128: 2.4}


def rope_angles(positions: torch.Tensor, inv_freq: torch.Tensor, pos_scale: float, rows: int, out: torch.Tensor) -> None:
    """out[r, i] = (cos, sin)(float(positions[r]) * pos_scale * inv_freq[i]): float32 [rows, len(inv_freq), 2]."""
    _cuda(positions, inv_freq, out)
    half = inv_freq.numel()
    if positions.dtype != torch.int32 or inv_freq.dtype != torch.float32 or out.dtype != torch.float32 \
            or out.numel() < rows * half * 2 or not out.is_contiguous() or out.data_ptr() % 16:
        raise InvalidArgument("rope_angles: int32 positions, float32 inv_freq, contiguous float32 out [rows, half, 2]")
    _check(_fn("rope_cache", "dl_rope_angles")(_p(positions), _p(inv_freq), half, pos_scale, rows, _p(out), _stream()),
           "rope_angles")


def gemm_qkv_rope(x: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                  row_request: torch.Tensor, block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  inv_freq: torch.Tensor, pos_scale: float, n_heads: int, n_kv_heads: int, head_dim: int,
                  page_size: int, angles: Optional[torch.Tensor] = None) -> None:
    """The q | k | v projection with rotary encoding and cache write in its epilogue: rotated q into
    q_out [rows, >= n_heads * head_dim], rotated k and plain v into the paged cache. The whole head is rotated
    (inv_freq has head_dim / 2 entries). bfloat16. Up to 16 rows: the weight-streaming kernel
    (csrc/gemm_skinny.cu, head_dim a multiple of 16); more rows: the tcgen05 kernel (csrc/gemm_tcgen05.cu,
    head_dim 64 or 128), which reads the step's (cos, sin) pairs from `angles` (see rope_angles) when given."""
    _cuda(x, w_qkv, q_out, positions, row_request, block_table, k_cache, v_cache, inv_freq)
    _rows_contiguous(x, "x")
    _rows_contiguous(q_out, "q_out")
    M, K = x.shape
    if any(t.dtype != torch.bfloat16 for t in (x, w_qkv, q_out, k_cache, v_cache)):
        raise Unsupported("gemm_qkv_rope: bfloat16 only")
    few = M <= SKINNY_FAST_ROWS
    if K % 8 or x.stride(0) % 8 or (head_dim % 16 if few else head_dim not in QKV_ROPE_TCGEN05_HEAD_DIMS):
        raise Unsupported(f"gemm_qkv_rope: {M} rows, K {K} and head_dim {head_dim}")
    if angles is not None and (angles.dtype != torch.float32 or angles.numel() < M * head_dim or not angles.is_contiguous()):
        raise InvalidArgument("gemm_qkv_rope: angles must be contiguous float32 [rows, head_dim / 2, 2]")
    if not few and (x.data_ptr() % 16 or w_qkv.data_ptr() % 16 or q_out.data_ptr() % 16 or q_out.stride(0) % 8):
        raise Unsupported("gemm_qkv_rope: x, w and q_out rows must be 16-byte aligned")
    if tuple(w_qkv.shape) != ((n_heads + 2 * n_kv_heads) * head_dim, K) or not w_qkv.is_contiguous():
        raise InvalidArgument("gemm_qkv_rope: w must be contiguous [(heads + 2 kv_heads) * head_dim, K]")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() * 2 != head_dim:
        raise Unsupported("gemm_qkv_rope: the rotary width must be the whole head (inv_freq float32 [head_dim / 2])")
    if q_out.shape[0] < M or q_out.shape[1] < n_heads * head_dim:
        raise InvalidArgument("gemm_qkv_rope: q_out is smaller than [rows, heads * head_dim]")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or k_cache.shape != v_cache.shape \
            or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise InvalidArgument("gemm_qkv_rope: cache shape is not [pages, page_size, kv_heads, head_dim]")
    if block_table.dtype != torch.int32 or block_table.stride(-1) != 1 or positions.dtype != torch.int32 \
            or row_request.dtype != torch.int32:
        raise InvalidArgument("gemm_qkv_rope: positions, row_request and block_table must be int32")
    if not few:
        library, name = (("gemm_tcgen05_cluster", "dl_gemm_tcgen05_cluster_qkv_rope") if tcgen05_pairs(M, w_qkv.shape[0])
                         else ("gemm_tcgen05", "dl_gemm_tcgen05_qkv_rope"))
        check_limits(library, pages=k_cache.shape[0], requests=block_table.shape[0], rows=M)
        _check(_fn(library, name)(
            _p(x), x.stride(0), _p(w_qkv), _p(q_out), q_out.stride(0), M, K, _p(positions), _p(row_request),
            _p(block_table), block_table.stride(0), _p(k_cache), _p(v_cache), _p(inv_freq), _p(angles), pos_scale, n_heads,
            n_kv_heads, head_dim, page_size, _p(_status_word(x.device)), _stream()), "gemm_tcgen05_qkv_rope")
        return
    check_limits("gemm_skinny", pages=k_cache.shape[0], requests=block_table.shape[0], rows=M)
    _check(_fn("gemm_skinny", "dl_gemm_skinny_qkv_rope")(
        _p(x), x.stride(0), _p(w_qkv), _p(q_out), q_out.stride(0), M, K, _p(positions), _p(row_request), _p(block_table),
        block_table.stride(0), _p(k_cache), _p(v_cache), _p(inv_freq), pos_scale, n_heads, n_kv_heads, head_dim, page_size,
        _stream()), "gemm_skinny_qkv_rope")


_tcgen05_status = {}
_pairs: Optional[bool] = None      # whether the variant with pairs of blocks sharing W tiles can be used


# rounds of 128 x 256 tiles over the SMs from which sharing W tiles between two blocks pays (measured on B200)
PAIRS_MIN_WAVES = float(os.environ.get("DYNALM_GEMM_PAIRS_MIN_WAVES", "4"))


def tcgen05_pairs(rows: int, features: int) -> bool:
    """Large products run the tcgen05 kernel in which two thread blocks share each tile of W
    (csrc/gemm_tcgen05_cluster.cu: 108 us against 119 us for 2048 x 16384 x 2048, 423 against 454 for 8192 rows),
    unless DYNALM_GEMM_PAIRS=0 or that source file is not there; smaller ones, where the pairing only couples the
    blocks' pipelines (54 us against 52 us for 2048 x 2048 x 8192), run csrc/gemm_tcgen05.cu."""
    global _pairs
    if _pairs is None:
        _pairs = os.environ.get("DYNALM_GEMM_PAIRS", "1") != "0" and \
            os.path.isfile(os.path.join(_lib.CSRC, "gemm_tcgen05_cluster.cu"))
    from .device import sm_count
    return _pairs and -(-rows // 128) * -(-features // 256) >= PAIRS_MIN_WAVES * sm_count()


def _status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device that the tcgen05 kernels write a code into when a wait inside them times out."""
    status = _tcgen05_status.get(device)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=device)
        _tcgen05_status[device] = status
    return status


def gemm_tcgen05_status(device=None) -> int:
    """The timeout code the tcgen05 kernels (matrix product, prompt attention) left on `device` (0: none).
    Reading it synchronises."""
    if device is None:
        return max((int(t.item()) for t in _tcgen05_status.values()), default=0)
    t = _tcgen05_status.get(torch.device(device))
    return 0 if t is None else int(t.item())


PREFILL_TCGEN05_HEAD_DIMS = (64, 128)


def paged_attention_prefill_tcgen05(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                                    q_tiles: torch.Tensor, n_tiles: int, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                                    head_dim: int, page_size: int, scale: float, window: int = 0,
                                    unit_parts: Optional[torch.Tensor] = None, partial: Optional[torch.Tensor] = None,
                                    counters: Optional[torch.Tensor] = None) -> None:
    """Flash attention of query tiles over the paged cache on tcgen05 tensor cores, bfloat16, head_dim 64 or
    128, pages of at least 16 keys; see csrc/attention_prefill_tcgen05.cu. Arguments as paged_attention_prefill.

    unit_parts: int32 [n_tiles], when the keys of some tiles are dealt over several entries of q_tiles (see
    kernels/attention.QueryTileParts): part | parts << 8 | scratch slot << 16 per entry, 0 = whole. Then partial:
    float32, (slots in use) * n_heads * (head_dim + 2) * 128 elements; counters: int32, (slots in use) * n_heads, zero."""
    _cuda(q, k_cache, v_cache, block_table, q_tiles, out, unit_parts, partial, counters)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise Unsupported("prefill attention (tcgen05): bfloat16 only")
    if head_dim not in PREFILL_TCGEN05_HEAD_DIMS or page_size < 16 or page_size & (page_size - 1) or n_heads % n_kv_heads:
        raise Unsupported(f"prefill attention (tcgen05): head_dim {head_dim} (64 or 128), page size {page_size} "
                          f"(a power of two from 16), heads {n_heads}:{n_kv_heads}")
    if (q.stride(0) % 8 or out.stride(0) % 8 or q.data_ptr() % 16 or out.data_ptr() % 16 or q_tiles.data_ptr() % 16
            or k_cache.data_ptr() % 16 or v_cache.data_ptr() % 16):
        raise Unsupported("prefill attention (tcgen05): q, out and cache rows must be 16-byte aligned")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or not k_cache.is_contiguous() or not v_cache.is_contiguous() \
            or v_cache.shape != k_cache.shape:
        raise InvalidArgument("prefill attention (tcgen05): cache shape is not [pages, page_size, kv_heads, head_dim]")
    if q_tiles.dtype != torch.int32 or q_tiles.numel() < 4 * n_tiles:
        raise InvalidArgument("prefill attention (tcgen05): q_tiles must be int32 [n_tiles, 4]")
    records = 0
    if unit_parts is not None:
        if unit_parts.dtype != torch.int32 or unit_parts.numel() < n_tiles or partial is None or counters is None \
                or partial.dtype != torch.float32 or counters.dtype != torch.int32:
            raise InvalidArgument("prefill attention (tcgen05): unit_parts int32 [n_tiles] with float32 partial and int32 counters")
        records = min(partial.numel() // (n_heads * (head_dim + 2) * 128), counters.numel() // n_heads)
        _status_companions.setdefault(q.device, {})[counters.data_ptr()] = counters
    check_limits("attention_prefill_tcgen05", pages=k_cache.shape[0], requests=block_table.shape[0], rows=q.shape[0])
    _check(_fn("attention_prefill_tcgen05", "dl_paged_attention_prefill_tcgen05")(
        _p(q), q.stride(0), q.shape[0], _p(k_cache), _p(v_cache), k_cache.shape[0], _p(block_table), block_table.stride(0),
        _p(q_tiles), n_tiles, _p(out), out.stride(0), n_heads, n_kv_heads, head_dim, page_size, scale, window,
        _p(_status_word(q.device)), _p(unit_parts), _p(partial), _p(counters), records, _stream()),
        "paged_attention_prefill_tcgen05")


def paged_attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                            q_tiles: torch.Tensor, n_tiles: int, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                            head_dim: int, page_size: int, scale: float, window: int = 0) -> None:
    """Flash attention of query tiles over the paged cache, bfloat16; see csrc/attention_prefill.cu.
    q_tiles: int32 [n_tiles, 4] = (request, first row, rows <= 128, first position)."""
    _cuda(q, k_cache, v_cache, block_table, q_tiles, out)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise Unsupported("prefill attention: bfloat16 only")
    if head_dim % 16 or head_dim > 128 or page_size & (page_size - 1) or n_heads % n_kv_heads:
        raise Unsupported(f"prefill attention: head_dim {head_dim} (multiple of 16 up to 128), page size {page_size} "
                          f"(a power of two), heads {n_heads}:{n_kv_heads}")
    if q.stride(0) % 8 or out.stride(0) % 2 or q.data_ptr() % 16 or out.data_ptr() % 4 or q_tiles.data_ptr() % 16:
        raise Unsupported("prefill attention: q rows must be 16-byte aligned, out rows 4-byte aligned")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise InvalidArgument("prefill attention: cache shape is not [pages, page_size, kv_heads, head_dim]")
    if q_tiles.dtype != torch.int32 or q_tiles.numel() < 4 * n_tiles:
        raise InvalidArgument("prefill attention: q_tiles must be int32 [n_tiles, 4]")
    check_limits("attention_prefill", pages=k_cache.shape[0], requests=block_table.shape[0], rows=q.shape[0])
    _check(_fn("attention_prefill", "dl_paged_attention_prefill")(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), block_table.stride(0), _p(q_tiles), n_tiles,
        _p(out), out.stride(0), n_heads, n_kv_heads, head_dim, page_size, scale, window, _stream()),
        "paged_attention_prefill")


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
              out_scale: float = 1.0) -> None:
    """out = (x @ w.T + bias) * out_scale with fp32 accumulation in a fixed order; see csrc/gemm_simt.cu."""
    _cuda(x, w, out, bias)
    _rows_contiguous(x, "x")
    _rows_contiguous(out, "out")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or out.shape != (M, N) or x.dtype != w.dtype:
        raise InvalidArgument("gemm: x [M, K], w [N, K] contiguous and of x's dtype, out [M, N]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise InvalidArgument("gemm: bias must be float32 [N]")
    _check(_fn("gemm_simt", "dl_gemm_simt")(dtype_code(x.dtype), dtype_code(out.dtype), _p(x), x.stride(0), _p(w),
                                             _p(bias), _p(out), out.stride(0), M, N, K, out_scale, _stream()), "gemm_simt")


SKINNY_MAX_ROWS = 64      # what the kernel takes
SKINNY_FAST_ROWS = int(os.environ.get("DYNALM_SKINNY_ROWS", "16"))     # up to here the dispatchers use it (measured on B200)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str = "store", out_scale: float = 1.0) -> None:
    """Weight-streaming product for at most 64 rows, bfloat16 operands; see csrc/gemm_skinny.cu.

    mode "store": out [M, N] bfloat16 or float32, or float32 [parts, M, N] to split K over `parts`
    blocks (the consumer adds the parts); mode "swiglu": w = [gate; up], out [M, N/2] bfloat16; mode "relu2":
    out [M, N] bfloat16 = max(x W^T, 0)^2."""
    _cuda(x, w, out)
    _rows_contiguous(x, "x")
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or w.shape[1] != K:
        raise InvalidArgument("gemm_skinny: x and w bfloat16, w [N, K] contiguous")
    if mode in ("relu2", "gelu_tanh") and (out.dim() != 2 or out.dtype != torch.bfloat16):
        raise InvalidArgument("gemm_skinny: an activation needs out [M, N] bfloat16")
    if M > SKINNY_MAX_ROWS or K % 8 or x.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16:
        raise Unsupported(f"gemm_skinny: at most {SKINNY_MAX_ROWS} rows, K a multiple of 8, 16-byte aligned rows")
    n_split, split_stride = 1, 0
    if mode == "swiglu":
        if N % 2 or out.shape != (M, N // 2) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
            raise InvalidArgument("gemm_skinny: swiglu needs out [M, N/2] bfloat16")
        code, ldy = 2, out.stride(0)
    elif out.dim() == 3:
        if out.dtype != torch.float32 or out.shape[1:] != (M, N) or not out.is_contiguous():
            raise InvalidArgument("gemm_skinny: split output must be contiguous float32 [parts, M, N]")
        code, ldy, n_split, split_stride = 1, N, out.shape[0], out.stride(0)
    else:
        if out.shape != (M, N) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
            raise InvalidArgument("gemm_skinny: out [M, N] bfloat16 or float32")
        code, ldy = (0 if out.dtype == torch.bfloat16 else 1), out.stride(0)
        if mode in ("relu2", "gelu_tanh"):
            code = 4 if mode == "relu2" else 5
    ahead, ahead_bytes = _take_ahead()
    _check(_fn("gemm_skinny", "dl_gemm_skinny")(_p(x), x.stride(0), _p(w), _p(out), ldy, M, N, K, code, out_scale,
                                                 n_split, split_stride, ahead, ahead_bytes, _stream()), "gemm_skinny")


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str = "store", out_scale: float = 1.0) -> None:
    """x W^T on tcgen05 tensor cores with TMA-fed operands; see csrc/gemm_tcgen05.cu.

    x [M, K] and w [N, K] bfloat16; out [M, N] bfloat16 or float32, or with mode "swiglu"
    (w = [gate; up]) out [M, N/2] bfloat16, or with mode "relu2" out [M, N] bfloat16 = max(x W^T, 0)^2."""
    _cuda(x, w, out)
    _rows_contiguous(x, "x")
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or w.shape[1] != K:
        raise InvalidArgument("gemm_tcgen05: x and w bfloat16, w [N, K] contiguous")
    if K % 8 or x.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or out.data_ptr() % 16 or out.stride(1) != 1:
        raise Unsupported("gemm_tcgen05: K and row pitches must be multiples of 8 elements, bases 16-byte aligned")
    if mode == "swiglu":
        if N % 16 or out.shape != (M, N // 2) or out.dtype != torch.bfloat16 or out.stride(0) % 8:
            raise Unsupported("gemm_tcgen05: swiglu needs out [M, N/2] bfloat16 with N/2 a multiple of 8")
        code = 2
    else:
        if out.shape != (M, N):
            raise InvalidArgument("gemm_tcgen05: out [M, N]")
        if out.dtype == torch.bfloat16:
            if N % 8 or out.stride(0) % 8:
                raise Unsupported("gemm_tcgen05: bfloat16 output needs N and its row pitch to be multiples of 8")
            code = 4 if mode == "relu2" else (5 if mode == "gelu_tanh" else 0)
        elif out.dtype == torch.float32 and mode not in ("relu2", "gelu_tanh"):
            if N % 4 or out.stride(0) % 4:
                raise Unsupported("gemm_tcgen05: float32 output needs N and its row pitch to be multiples of 4")
            code = 1
        else:
            raise InvalidArgument("gemm_tcgen05: out bfloat16 or float32")
    status = _status_word(x.device)
    library, name = (("gemm_tcgen05_cluster", "dl_gemm_tcgen05_cluster") if tcgen05_pairs(M, N)
                     else ("gemm_tcgen05", "dl_gemm_tcgen05"))
    _check(_fn(library, name)(_p(x), x.stride(0), _p(w), _p(out), out.stride(0), M, N, K, code, out_scale, _p(status),
                              _stream()), "gemm_tcgen05")


def gemm_tcgen05_tile_coords(tile: int, tiles_n: int, num_tiles: int, group_m: int):
    """(row block, column block) of tile number `tile` in the tcgen05 product's numbering of num_tiles output tiles in
    tiles_n columns, groups of group_m row blocks (csrc/gemm_tcgen05_impl.cuh, t5_tile_coords). Runs on the host: it
    is there so that the numbering can be tested without a GPU."""
    from ctypes import byref, c_int
    m, n = c_int(-1), c_int(-1)
    _check(_fn("gemm_tcgen05", "dl_gemm_tcgen05_tile_coords")(tile, tiles_n, num_tiles, group_m, byref(m), byref(n)),
           "gemm_tcgen05_tile_coords")
    return m.value, n.value


STREAM_MAX_ROWS = 64       # what the tcgen05 weight-streaming product takes


def gemm_stream(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str = "store", out_scale: float = 1.0) -> None:
    """x W^T for up to 64 bfloat16 rows on tcgen05, built around the stream of W (csrc/gemm_stream_tcgen05.cu).

    out [M, N] bfloat16 or float32; float32 [parts, M, N] (contiguous): K is split over `parts` blocks and each
    leaves its partial sums; mode "swiglu" (w = [gate; up]): out [M, N/2] bfloat16; mode "relu2": out [M, N] bfloat16 =
    max(x W^T, 0)^2."""
    _cuda(x, w, out)
    _rows_contiguous(x, "x")
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or w.shape[1] != K:
        raise InvalidArgument("gemm_stream: x and w bfloat16, w [N, K] contiguous")
    if M > STREAM_MAX_ROWS or K % 8 or x.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16:
        raise Unsupported(f"gemm_stream: at most {STREAM_MAX_ROWS} rows, K a multiple of 8, 16-byte aligned rows")
    n_split, split_stride = 1, 0
    if mode == "swiglu":
        if N % 2 or out.shape != (M, N // 2) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
            raise InvalidArgument("gemm_stream: swiglu needs out [M, N/2] bfloat16")
        code, ldy = 2, out.stride(0)
    elif out.dim() == 3:
        if out.dtype != torch.float32 or out.shape[1:] != (M, N) or not out.is_contiguous():
            raise InvalidArgument("gemm_stream: split output must be contiguous float32 [parts, M, N]")
        code, ldy, n_split, split_stride = 1, N, out.shape[0], out.stride(0)
    else:
        if out.shape != (M, N) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
            raise InvalidArgument("gemm_stream: out [M, N] bfloat16 or float32")
        code, ldy = (0 if out.dtype == torch.bfloat16 else 1), out.stride(0)
        if mode in ("relu2", "gelu_tanh"):
            if out.dtype != torch.bfloat16:
                raise InvalidArgument("gemm_stream: an activation needs out [M, N] bfloat16")
            code = 3 if mode == "relu2" else 4
    _check(_fn("gemm_stream_tcgen05", "dl_gemm_stream")(
        _p(x), x.stride(0), _p(w), _p(out), ldy, M, N, K, code, out_scale, n_split, split_stride,
        _p(_status_word(x.device)), _stream()), "gemm_stream")


_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor, status_to: Optional[torch.Tensor] = None) -> None:
    """out[r] = lowest index of the largest value of logits[r, :] (float32 rows, int32 out). `status_to` (int32, one
    element): also receives the device's status word (see gemm_tcgen05_status), so that it can travel to the host
    in the copy that carries the chosen ids."""
    _cuda(logits, out)
    _rows_contiguous(logits, "logits")
    rows = logits.shape[0]
    if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() < rows:
        raise InvalidArgument("argmax: logits float32, out int32 with one entry per row")
    # partial (value, index) pairs of the two-stage kernel; grown in powers of two, kept per device
    key = logits.device
    scratch = _argmax_scratch.get(key)
    if scratch is None or scratch.numel() < rows * 64:
        scratch = torch.empty(max(64, 1 << (rows * 64 - 1).bit_length()), dtype=torch.float32, device=logits.device)
        _argmax_scratch[key] = scratch
    status = _status_word(logits.device) if status_to is not None else None
    _check(_fn("sampling", "dl_argmax")(_p(logits), logits.stride(0), rows, logits.shape[1], _p(out), _p(scratch),
                                         _p(status), _p(status_to), _stream()), "argmax")


_status_companions: dict = {}      # device -> {address: counters that a kernel leaves nonzero only when a wait timed out}


def clear_status(device) -> None:
    """Zero the device's status word after its code has been reported, and the counters that a kernel which gave up
    may have left half counted (the prompt attention's parts)."""
    t = _tcgen05_status.get(torch.device(device))
    if t is not None:
        t.zero_()
    for counters in _status_companions.get(torch.device(device), {}).values():
        counters.zero_()


def zero_pages(storage: torch.Tensor, fresh: torch.Tensor, n: int, group: int) -> None:
    """Clear the pages listed for `group` in the first n pairs (group id, page) of `fresh` (int32) in every array of a
    cache group's storage [entries, tensors, pages, page_size, ...] (csrc/table_update.cu)."""
    _cuda(storage, fresh)
    if not storage.is_contiguous() or storage.dim() < 4 or fresh.dtype != torch.int32 or fresh.numel() < 2 * n:
        raise InvalidArgument("zero_pages: contiguous storage [entries, tensors, pages, ...] and int32 pairs")
    pages = storage.shape[2]
    page_bytes = storage[0, 0, 0].numel() * storage.element_size()
    _check(_fn("table_update", "dl_zero_pages")(_p(storage), page_bytes, pages, storage.shape[0] * storage.shape[1], _p(fresh),
                                                 n, group, _stream()), "zero_pages")


def table_updates(tables: torch.Tensor, updates: torch.Tensor, n: int) -> None:
    """tables[g, s, b] = p for the first n quadruples (g, s, b, p) of `updates` (csrc/table_update.cu): the
    device's block tables [groups, slots, max_blocks], int32, brought up to date with what a step changed."""
    _cuda(tables, updates)
    if tables.dtype != torch.int32 or updates.dtype != torch.int32 or tables.dim() != 3 or not tables.is_contiguous() \
            or updates.numel() < 4 * n or updates.data_ptr() % 16:
        raise InvalidArgument("table_updates: int32 tables [groups, slots, blocks] and int32 updates [n, 4], 16-byte aligned")
    check_limits("table_update", requests=tables.shape[1])
    _check(_fn("table_update", "dl_table_updates")(_p(tables), _p(updates), n, tables.shape[0], tables.shape[1],
                                                    tables.shape[2], _stream()), "table_updates")


def gemm_argmax_applies(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether `gemm_argmax` takes this product: the weight-streaming kernel's shapes, up to 8 rows."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] <= 8 and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous()
            and w.data_ptr() % 16 == 0)


def gemm_argmax(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, out_scale: float = 1.0,
                status_to: Optional[torch.Tensor] = None) -> None:
    """out[r] = the index of the largest element of (x W^T)[r] * out_scale, the lowest among equals, without the
    product ever being written: the weight-streaming kernel leaves one candidate per block (csrc/gemm_skinny.cu,
    mode 3) and a small kernel picks among them. `scratch`: float32, at least 2 * rows * ceil(N / 16) elements.
    out_scale must be positive. `status_to` as in `argmax`."""
    _cuda(x, w, out, scratch)
    if not gemm_argmax_applies(x, w) or w.shape[1] != x.shape[1] or out_scale <= 0:
        raise Unsupported("gemm_argmax: up to 8 bfloat16 rows, K a multiple of 8, 16-byte aligned rows, a positive scale")
    M, K = x.shape
    N = w.shape[0]
    blocks = -(-N // 16)
    if scratch.dtype != torch.float32 or scratch.numel() < 2 * M * blocks or out.dtype != torch.int32 or out.numel() < M:
        raise InvalidArgument("gemm_argmax: float32 scratch of 2 * rows * ceil(N / 16) elements, int32 out of one per row")
    ahead, ahead_bytes = _take_ahead()
    _check(_fn("gemm_skinny", "dl_gemm_skinny")(_p(x), x.stride(0), _p(w), _p(scratch), blocks, M, N, K, 3, out_scale,
                                                 1, 0, ahead, ahead_bytes, _stream()), "gemm_skinny (argmax)")
    status = _status_word(x.device) if status_to is not None else None
    _check(_fn("sampling", "dl_argmax_of_parts")(_p(scratch), scratch.data_ptr() + 4 * M * blocks, M, blocks, _p(out),
                                                  _p(status), _p(status_to), _stream()), "argmax_of_parts")


def feedback_tokens(token_ids: torch.Tensor, chosen: torch.Tensor, src: torch.Tensor, n: int) -> None:
    """token_ids[r] = chosen[src[r]] for r < n where src[r] >= 0 (all int32, on the device)."""
    _cuda(token_ids, chosen, src)
    if token_ids.dtype != torch.int32 or chosen.dtype != torch.int32 or src.dtype != torch.int32 or min(token_ids.numel(), src.numel()) < n:
        raise InvalidArgument("feedback_tokens: int32 tensors with at least n entries")
    check_limits("sampling", rows=chosen.numel())
    _check(_fn("sampling", "dl_feedback_tokens")(_p(token_ids), _p(chosen), _p(src), n, _stream()), "feedback_tokens")


def sample_temperature(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor,
                       cut_offset: Optional[torch.Tensor] = None) -> None:
    """Draw out[r] from softmax(logits[r] / temperature[r]) by walking the ids in order with uniform[r]. With
    cut_offset (float64 [rows]: temperature * log(min_p), -inf where off) the ids whose logit lies below the row's
    largest plus the offset have no mass (min-p)."""
    _cuda(logits, temperature, uniform, out, cut_offset)
    _rows_contiguous(logits, "logits")
    rows = logits.shape[0]
    if (logits.dtype != torch.float32 or temperature.dtype != torch.float32 or uniform.dtype != torch.float64
            or out.dtype != torch.int32 or min(temperature.numel(), uniform.numel(), out.numel()) < rows):
        raise InvalidArgument("sample_temperature: logits/temperature float32, uniform float64, out int32, one per row")
    if cut_offset is not None and (cut_offset.dtype != torch.float64 or cut_offset.numel() < rows):
        raise InvalidArgument("sample_temperature: cut_offset float64, one per row")
    _check(_fn("sampling", "dl_sample_temperature")(_p(logits), logits.stride(0), rows, logits.shape[1], _p(temperature),
                                                     _p(uniform), _p(cut_offset), _p(out), _stream()), "sample_temperature")


def apply_penalties(logits: torch.Tensor, rows: torch.Tensor, triples: torch.Tensor, n_triples: int,
                    params: torch.Tensor, first: torch.Tensor, chosen: Optional[torch.Tensor] = None,
                    pending: Optional[torch.Tensor] = None) -> None:
    """Repetition, frequency and presence penalties, in place: triple j = (selection, token id, count) changes
    logits[rows[selection], id] with params[selection] = (repetition, frequency, presence). The ids of one selection
    are distinct and its triples lie next to one another, from first[selection] to first[selection + 1]. rows int32
    [selections], triples int32 [>= n_triples, 3], params float32 [selections, 3], first int32 [selections + 1].
    chosen and pending (int32, both or neither): pending[selection] >= 0 is the place in `chosen` of one more token
    of that selection's context, which only the device knows yet; it counts as seen once more."""
    _cuda(logits, rows, triples, params, first, chosen, pending)
    _rows_contiguous(logits, "logits")
    n_sel = rows.numel()
    if (logits.dtype != torch.float32 or rows.dtype != torch.int32 or triples.dtype != torch.int32
            or params.dtype != torch.float32 or first.dtype != torch.int32 or triples.numel() < 3 * n_triples
            or not triples.is_contiguous() or not params.is_contiguous() or params.numel() < 3 * n_sel
            or first.numel() < n_sel + 1):
        raise InvalidArgument("apply_penalties: logits/params float32, rows/triples/first int32, triples [n, 3]")
    if (chosen is None) != (pending is None) or (pending is not None and (
            pending.dtype != torch.int32 or chosen.dtype != torch.int32 or pending.numel() < n_sel)):
        raise InvalidArgument("apply_penalties: chosen and pending int32, together, pending one per selection")
    if CHECKED:
        check_limits("sampling", rows=logits.shape[0])
    _check(_fn("sampling", "dl_apply_penalties")(_p(logits), logits.stride(0), logits.shape[1], _p(rows), _p(triples),
                                                  int(n_triples), _p(params), _p(first), n_sel, _p(chosen), _p(pending),
                                                  _stream()), "apply_penalties")


SAMPLE_FILTERED_HOST = -1      # what sample_filtered leaves for a row that the host has to finish


def sample_filtered(logits: torch.Tensor, rows: torch.Tensor, n_sel: int, dparams: torch.Tensor, top_k: torch.Tensor,
                    out: torch.Tensor) -> None:
    """One draw per selection through top-k, min-p and top-p in the reference's order. rows int32 [n_sel]: the
    logits row of each selection; dparams float64 [n_sel, 4] = (temperature, temperature * log(min_p) or -inf, top_p,
    uniform in [0, 1)); top_k int32 [n_sel] (0 = off); out int32 with a place for every row named: out[rows[sel]] gets the id,
    or SAMPLE_FILTERED_HOST where the row does not fit the kernel (top-k above 1,024, say)."""
    _cuda(logits, rows, dparams, top_k, out)
    _rows_contiguous(logits, "logits")
    if (logits.dtype != torch.float32 or rows.dtype != torch.int32 or dparams.dtype != torch.float64
            or top_k.dtype != torch.int32 or out.dtype != torch.int32 or not dparams.is_contiguous()
            or min(rows.numel(), top_k.numel(), out.numel()) < n_sel or dparams.numel() < 4 * n_sel):
        raise InvalidArgument("sample_filtered: logits float32, rows/top_k/out int32, dparams float64 [n, 4]")
    if CHECKED:
        check_limits("sampling", rows=min(logits.shape[0], out.numel()))      # a row is also a place in `out`
    _check(_fn("sampling", "dl_sample_filtered")(_p(logits), logits.stride(0), logits.shape[1], _p(rows), int(n_sel),
                                                  _p(dparams), _p(top_k), _p(out), _stream()), "sample_filtered")


# ---------------------------------------------------------------------------------------------
# short convolutions with options, the gated delta rule, the gated linear recurrence, whole-projection query/key norms,
# gates and caps

def _state_rows(state: torch.Tensor, need: int, what: str) -> None:
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < need:
        raise InvalidArgument(f"{what}: state float32 [slots, >= {need}]")


def short_conv(proj: torch.Tensor, col0: int, channels: int, taps_t: torch.Tensor, bias: Optional[torch.Tensor],
               state: torch.Tensor, keep_off: int, positions: torch.Tensor, row_request: torch.Tensor,
               row_slot: torch.Tensor, pos_start: torch.Tensor, out: torch.Tensor, act: str = "silu",
               in_bias: Optional[torch.Tensor] = None) -> None:
    """ssm_conv with its options: act "silu" or "none" on the result; in_bias (float32 [channels]) joins every input
    that lies inside the sequence before the taps (kept inputs are stored without it). See csrc/ssm.cu."""
    taps = taps_t
    _cuda(proj, taps, bias, state, positions, row_request, row_slot, pos_start, out, in_bias)
    _rows_contiguous(proj, "proj")
    rows, K = proj.shape[0], taps.shape[0]
    if act not in ("silu", "none"):
        raise InvalidArgument(f"short_conv: no activation '{act}' (silu, none)")
    if taps.dtype != torch.float32 or not taps.is_contiguous() or taps.dim() != 2 or taps.shape[1] != channels:
        raise InvalidArgument("short_conv: taps float32 [K, channels]")
    for b in (bias, in_bias):
        if b is not None and (b.dtype != torch.float32 or b.numel() != channels):
            raise InvalidArgument("short_conv: a bias is float32 [channels]")
    _state_rows(state, keep_off + (K - 1) * channels, "short_conv")
    if out.dtype != proj.dtype or out.shape != (rows, channels) or not out.is_contiguous() or col0 + channels > proj.shape[1]:
        raise InvalidArgument("short_conv: out contiguous [rows, channels] of proj's dtype; the channels lie inside proj")
    check_limits("ssm", requests=state.shape[0], rows=rows)
    _check(_fn("ssm", "dl_short_conv")(dtype_code(proj.dtype), _p(proj), proj.stride(0), col0, channels, _p(taps), _p(bias), K,
                                        _p(state), state.stride(0), keep_off, _p(positions), _p(row_request), _p(row_slot),
                                        _p(pos_start), _p(out), rows, 1 if act == "silu" else 0, _p(in_bias), _stream()),
           "short_conv")


def delta_rule(u: torch.Tensor, q_col: int, k_col: int, v_col: int, proj: torch.Tensor, b_col: int, a_col: int,
               a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor,
               state_slots: torch.Tensor, out: torch.Tensor, requests: int, heads: int, kv_heads: int, dim: int,
               vdim: int) -> None:
    """The gated delta rule of every head over every request's rows of the step, from and into state[slot, :H*d*e]
    ([H, d, e]). u: rows with q (G*d) at q_col, k (G*d) at k_col, v (H*e) at v_col, after convolution and silu; proj:
    rows with the raw write strengths (H) at b_col and the raw step sizes (H) at a_col; out: float32 [rows, H*e].
    See csrc/delta_rule.cu."""
    _cuda(u, proj, a_log, dt_bias, state, q_start, state_slots, out)
    _rows_contiguous(u, "u")
    _rows_contiguous(proj, "proj")
    if u.dtype != proj.dtype or max(q_col, k_col) + kv_heads * dim > u.shape[1] or v_col + heads * vdim > u.shape[1] \
            or max(b_col, a_col) + heads > proj.shape[1]:
        raise InvalidArgument("delta_rule: the columns lie outside u or proj, or their dtypes differ")
    if any(t.dtype != torch.float32 or t.numel() != heads for t in (a_log, dt_bias)):
        raise InvalidArgument("delta_rule: a_log and dt_bias are float32 [heads]")
    if heads % kv_heads or dim > 512:
        raise Unsupported(f"delta_rule: {heads} heads over {kv_heads} query/key heads of {dim} (at most 512) has no kernel")
    _state_rows(state, heads * dim * vdim, "delta_rule")
    if out.dtype != torch.float32 or not out.is_contiguous() or out.shape != (u.shape[0], heads * vdim):
        raise InvalidArgument("delta_rule: out float32 contiguous [rows, H*e]")
    check_limits("delta_rule", requests=state.shape[0], rows=u.shape[0])
    # a step of single tokens goes to the light kernel that is bound by the state's trip through memory alone
    entry = "dl_delta_rule_step" if u.shape[0] <= requests else "dl_delta_rule"
    _check(_fn("delta_rule", entry)(dtype_code(u.dtype), _p(u), u.stride(0), q_col, k_col, v_col, _p(proj),
                                               proj.stride(0), b_col, a_col, _p(a_log), _p(dt_bias), _p(state),
                                               state.stride(0), _p(q_start), _p(state_slots), _p(out), requests, heads,
                                               kv_heads, dim, vdim, _stream()), "delta_rule")


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, gate_col: int, weight: torch.Tensor, eps: float, out: torch.Tensor,
                   heads: int, vdim: int) -> None:
    """out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * silu(gate[t, gate_col + h * e ...]).
    o: float32 contiguous [rows, H*e]; weight: float32 [e]; out: contiguous [rows, H*e] of gate's dtype."""
    _cuda(o, gate, weight, out)
    _rows_contiguous(gate, "gate")
    rows = o.shape[0]
    if o.dtype != torch.float32 or not o.is_contiguous() or o.shape != (rows, heads * vdim) or weight.dtype != torch.float32 \
            or weight.numel() != vdim or out.shape != o.shape or not out.is_contiguous() or out.dtype != gate.dtype \
            or gate_col + heads * vdim > gate.shape[1] or gate.shape[0] < rows:
        raise InvalidArgument("head_norm_gate: o float32 [rows, H*e], weight float32 [e], out [rows, H*e] of the gate's dtype")
    _check(_fn("delta_rule", "dl_head_norm_gate")(dtype_code(gate.dtype), _p(o), _p(gate), gate.stride(0), gate_col,
                                                   _p(weight), eps, _p(out), rows, heads, vdim, _stream()), "head_norm_gate")


def rglru_gates(u: torch.Tensor, wa_t: torch.Tensor, ba: torch.Tensor, wi_t: torch.Tensor, bi: torch.Tensor,
                lam: torch.Tensor, decay_scale: float, a_out: torch.Tensor, m_out: torch.Tensor) -> None:
    """Per row and channel the decay a and the gated input m of a real-gated linear recurrent unit. u: contiguous [rows,
    width]; wa_t, wi_t: float32 [blocks, in, out]; ba, bi, lam: float32 [width]; a_out, m_out: float32 [rows, width].
    See csrc/rglru.cu."""
    _cuda(u, wa_t, ba, wi_t, bi, lam, a_out, m_out)
    rows, width = u.shape
    blocks = wa_t.shape[0]
    nb = width // max(blocks, 1)
    if not u.is_contiguous() or any(t.dtype != torch.float32 or not t.is_contiguous() for t in (wa_t, ba, wi_t, bi, lam, a_out, m_out)) \
            or tuple(wa_t.shape) != (blocks, nb, nb) or wi_t.shape != wa_t.shape or blocks * nb != width \
            or any(t.numel() != width for t in (ba, bi, lam)) or a_out.shape != u.shape or m_out.shape != u.shape:
        raise InvalidArgument("rglru_gates: shapes or dtypes disagree")
    _check(_fn("rglru", "dl_rglru_gates")(dtype_code(u.dtype), _p(u), _p(wa_t), _p(ba), _p(wi_t), _p(bi), _p(lam),
                                           decay_scale, _p(a_out), _p(m_out), rows, width, blocks, _stream()), "rglru_gates")


def rglru_scan(a: torch.Tensor, m: torch.Tensor, y: torch.Tensor, y_col: int, y_bias: Optional[torch.Tensor],
               state: torch.Tensor, q_start: torch.Tensor, state_slots: torch.Tensor, out: torch.Tensor,
               requests: int) -> None:
    """S <- a S + m along every request's rows of the step, from and into state[slot, :width]; out = S *
    gelu_tanh(y[:, y_col ...] + y_bias). a, m: float32 [rows, width]; out: contiguous [rows, width] of y's dtype."""
    _cuda(a, m, y, y_bias, state, q_start, state_slots, out)
    _rows_contiguous(y, "y")
    rows, width = a.shape
    if a.dtype != torch.float32 or m.dtype != torch.float32 or not a.is_contiguous() or not m.is_contiguous() \
            or m.shape != a.shape or out.shape != a.shape or not out.is_contiguous() or out.dtype != y.dtype \
            or y_col + width > y.shape[1] or (y_bias is not None and (y_bias.dtype != torch.float32 or y_bias.numel() != width)):
        raise InvalidArgument("rglru_scan: shapes or dtypes disagree")
    _state_rows(state, width, "rglru_scan")
    check_limits("rglru", requests=state.shape[0], rows=rows)
    _check(_fn("rglru", "dl_rglru_scan")(dtype_code(y.dtype), _p(a), _p(m), _p(y), y.stride(0), y_col, _p(y_bias), _p(state),
                                          state.stride(0), _p(q_start), _p(state_slots), _p(out), requests, width, rows,
                                          _stream()), "rglru_scan")


def qk_proj_norm_cache(proj: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float, do_norm: bool,
                       inv_freq: Optional[torch.Tensor], rot: int, pos_scale: float, positions: torch.Tensor,
                       row_slot: torch.Tensor, block_table: torch.Tensor, k_cache: torch.Tensor, k_row: int,
                       v_cache: torch.Tensor, v_row: int, heads: int, kv_heads: int, dim: int, vdim: int,
                       page_size: int) -> None:
    """Rows [q: H*d | k: G*d | v: G*e | ...] of a projection: q and k normed over the whole projection (one statistic
    each, weights wq / wk), their heads' first `rot` numbers turned by position (pairs i, i + rot/2), q written back
    in place, k and v written to the token's place in the cache: k_cache / v_cache point at the first token's keys /
    values, k_row / v_row elements lie between two tokens. See csrc/qk_proj_norm.cu."""
    _cuda(proj, wq, wk, inv_freq, positions, row_slot, block_table, k_cache, v_cache)
    _rows_contiguous(proj, "proj")
    if proj.shape[1] < heads * dim + kv_heads * (dim + vdim) or k_cache.dtype != proj.dtype or v_cache.dtype != proj.dtype:
        raise InvalidArgument("qk_proj_norm_cache: proj holds q | k | v; the cache has proj's dtype")
    for w, n in ((wq, heads * dim), (wk, kv_heads * dim)):
        if w is not None and (w.dtype != torch.float32 or w.numel() != n):
            raise InvalidArgument("qk_proj_norm_cache: a norm weight is float32 over the whole projection")
    if rot and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() < rot // 2):
        raise InvalidArgument("qk_proj_norm_cache: inv_freq float32 [rot / 2]")
    check_limits("qk_proj_norm", pages=k_cache.shape[0], requests=block_table.shape[0], rows=proj.shape[0])
    _check(_fn("qk_proj_norm", "dl_qk_proj_norm_cache")(
        dtype_code(proj.dtype), _p(proj), proj.stride(0), _p(wq), _p(wk), eps, 1 if do_norm else 0, _p(inv_freq), rot,
        pos_scale, _p(positions), _p(row_slot), _p(block_table), block_table.stride(0), _p(k_cache), k_row, _p(v_cache),
        v_row, proj.shape[0], heads, kv_heads, dim, vdim, page_size, _stream()), "qk_proj_norm_cache")


def paged_attention_generic_kv(q: torch.Tensor, k_cache: torch.Tensor, k_row: int, v_cache: torch.Tensor, v_row: int,
                               block_table: torch.Tensor, positions: torch.Tensor, row_request: torch.Tensor,
                               out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, vdim: int, page_size: int,
                               scale: float, window: int = 0, keep_first: int = 0, sink: bool = False) -> None:
    """paged_attention_generic with keys of head_dim and values of vdim numbers: k_cache / v_cache point at the first
    token's keys / values (KV head j at j * head_dim / j * vdim), k_row / v_row elements lie between two tokens.
    out: rows with head h at column h * vdim. keep_first: keys at positions below it stay visible behind the window;
    sink: the softmax's denominator holds one more term of score 0, which carries no value."""
    _cuda(q, k_cache, v_cache, block_table, positions, row_request, out)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if not 0 < head_dim <= 256 or not 0 < vdim <= 256:
        raise Unsupported(f"attention: keys of {head_dim} and values of {vdim} numbers (at most 256 each)")
    if n_heads % n_kv_heads:
        raise Unsupported(f"attention: {n_heads} heads do not divide into {n_kv_heads} KV heads")
    if q.dtype != out.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise InvalidArgument("attention: q, out and the cache must share one dtype")
    check_limits("attention_generic", pages=k_cache.shape[0], requests=block_table.shape[0], rows=q.shape[0])
    _check(_fn("attention_generic", "dl_paged_attention_generic_masked")(
        dtype_code(q.dtype), _p(q), q.stride(0), _p(k_cache), k_row, _p(v_cache), v_row, _p(block_table),
        block_table.stride(0), _p(positions), _p(row_request), _p(out), out.stride(0), q.shape[0], n_heads, n_kv_heads,
        head_dim, vdim, page_size, scale, window, int(keep_first), 1 if sink else 0, _stream()), "paged_attention_generic_kv")


def gelu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = gelu_tanh(gate_up[t, j]) * gate_up[t, inner + j]."""
    _cuda(gate_up, out)
    rows, inner = out.shape
    if gate_up.shape != (rows, 2 * inner) or gate_up.dtype != out.dtype or not gate_up.is_contiguous() or not out.is_contiguous():
        raise InvalidArgument("gelu_mul: gate_up contiguous [rows, 2 * inner], out contiguous [rows, inner], one dtype")
    _check(_fn("gates", "dl_gelu_mul")(dtype_code(out.dtype), _p(gate_up), _p(out), rows, inner, _stream()), "gelu_mul")


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> None:
    """x[t, j] <- x[t, j] * sigmoid(gate[t, j]) over x's columns; both 2-D views with unit column stride."""
    _cuda(x, gate)
    _rows_contiguous(x, "x")
    _rows_contiguous(gate, "gate")
    if x.dtype != gate.dtype or gate.shape[0] < x.shape[0] or gate.shape[1] < x.shape[1]:
        raise InvalidArgument("sigmoid_gate: x and gate of one dtype, the gate at least as large as x")
    _check(_fn("gates", "dl_sigmoid_gate")(dtype_code(x.dtype), _p(x), x.stride(0), _p(gate), gate.stride(0), x.shape[0],
                                            x.shape[1], _stream()), "sigmoid_gate")


def scaled_sum(a: torch.Tensor, sa: float, b: torch.Tensor, sb: float, out: torch.Tensor) -> None:
    """out = sa * a + sb * b (float32 [n, width]); a and b are [n, width] or split-K partial sums [parts, n, width] of
    either dtype, added in order."""
    _cuda(a, b, out)
    width = out.shape[-1]
    pa, stride_a = _delta_parts(a, width, "scaled_sum")
    pb, stride_b = _delta_parts(b, width, "scaled_sum")
    if out.dtype != torch.float32 or not out.is_contiguous() or a.shape[-2:] != out.shape or b.shape[-2:] != out.shape:
        raise InvalidArgument("scaled_sum: out float32 contiguous, of the shape of a and b")
    _check(_fn("gates", "dl_scaled_sum")(dtype_code(a.dtype), _p(a), pa, stride_a, sa, dtype_code(b.dtype), _p(b), pb,
                                          stride_b, sb, _p(out), out.numel(), _stream()), "scaled_sum")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place; x float32 contiguous."""
    _cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise InvalidArgument("softcap: x float32 contiguous")
    _check(_fn("gates", "dl_softcap")(_p(x), x.numel(), cap, _stream()), "softcap")


def norm_add_norm(x: torch.Tensor, delta: torch.Tensor, w_post: torch.Tensor, eps_post: float,
                  w_pre: Optional[torch.Tensor] = None, eps_pre: float = 0.0, out: Optional[torch.Tensor] = None) -> None:
    """x <- x + rmsnorm(delta) * w_post, then (with w_pre) out = rmsnorm(x) * w_pre. x: float32 [n, width] in place;
    delta: [n, width] of either dtype or partial sums [parts, n, width]; out: [n, width]. See csrc/norm_sandwich.cu."""
    _cuda(x, delta, w_post, w_pre, out)
    rows, width = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or w_post.dtype != torch.float32 or w_post.numel() != width:
        raise InvalidArgument("norm_add_norm: x float32 contiguous, w_post float32 [width]")
    if (w_pre is None) != (out is None) or (w_pre is not None and (w_pre.dtype != torch.float32 or w_pre.numel() != width
                                                                  or out.shape != x.shape or not out.is_contiguous())):
        raise InvalidArgument("norm_add_norm: w_pre float32 [width] together with out contiguous [n, width], or neither")
    parts, part_stride = _delta_parts(delta, width, "norm_add_norm")
    if delta.shape[-2] < rows:
        raise InvalidArgument("norm_add_norm: delta has fewer rows than x")
    od = dtype_code(out.dtype) if out is not None else 0
    _take_ahead()
    _check(_fn("norm_sandwich", "dl_norm_add_norm")(od, dtype_code(delta.dtype), _p(x), _p(delta), parts, part_stride,
                                                     _p(w_post), eps_post, _p(w_pre), eps_pre, _p(out), rows, width,
                                                     _stream()), "norm_add_norm")


def qk_rot_head_norm_cache(proj: torch.Tensor, inv_freq: Optional[torch.Tensor], rot: int, interleaved: bool, unit_norm: bool,
                           eps: float, positions: torch.Tensor, row_slot: torch.Tensor, block_table: torch.Tensor,
                           k_cache: torch.Tensor, k_row: int, v_cache: torch.Tensor, v_row: int, heads: int, kv_heads: int,
                           dim: int, vdim: int, page_size: int, bias: Optional[torch.Tensor] = None) -> None:
    """Rows [q: H*d | k: G*d | v: G*e | ...] of a projection (plus `bias`, float32 over q | k | v, when given): the first `rot` numbers of every head of q and k turned by
    position (pairs i, i + rot/2, or 2i, 2i + 1 when interleaved), then every head divided by its own root mean square
    (unit_norm) or left; q written back in place, k and v written to the token's place in the cache (k_cache / v_cache
    point at the first token's keys / values, k_row / v_row elements lie between two tokens). See csrc/qk_proj_norm.cu."""
    _cuda(proj, inv_freq, positions, row_slot, block_table, k_cache, v_cache)
    _rows_contiguous(proj, "proj")
    if proj.shape[1] < heads * dim + kv_heads * (dim + vdim) or k_cache.dtype != proj.dtype or v_cache.dtype != proj.dtype:
        raise InvalidArgument("qk_rot_head_norm_cache: proj holds q | k | v; the cache has proj's dtype")
    if dim > 256:
        raise Unsupported(f"qk_rot_head_norm_cache: heads of {dim} numbers (256 at most)")
    if rot and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() < rot // 2):
        raise InvalidArgument("qk_rot_head_norm_cache: inv_freq float32 [rot / 2]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() < heads * dim + kv_heads * (dim + vdim)):
        raise InvalidArgument("qk_rot_head_norm_cache: bias float32 over q | k | v")
    _cuda(bias)
    check_limits("qk_proj_norm", pages=k_cache.shape[0], requests=block_table.shape[0], rows=proj.shape[0])
    _check(_fn("qk_proj_norm", "dl_qk_rot_head_norm_cache")(
        dtype_code(proj.dtype), _p(proj), proj.stride(0), _p(bias), _p(inv_freq), rot, 1 if interleaved else 0, 1 if unit_norm else 0,
        eps, _p(positions), _p(row_slot), _p(block_table), block_table.stride(0), _p(k_cache), k_row, _p(v_cache), v_row,
        proj.shape[0], heads, kv_heads, dim, vdim, page_size, _stream()), "qk_rot_head_norm_cache")


STREAM_MAX_PARTS = 16      # the most parts a residual stream may have (csrc/layer_norm.cu)


def stream_layer_norm(streams: torch.Tensor, parts: int, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float,
                      out: Optional[torch.Tensor], init: Optional[torch.Tensor] = None, delta: Optional[torch.Tensor] = None,
                      delta_scale: float = 1.0, mix: Optional[torch.Tensor] = None, write: Optional[torch.Tensor] = None,
                      read: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                      n_rows: Optional[int] = None) -> None:
    """Layer norm over a residual stream of `parts` parts, fused with the update the sublayer in front left pending.

    streams: float32 [n, parts * width] (a row's parts one after the other), updated in place unless `rows` gathers.
    init [n, width] float32: every part of a row starts as this row (the first layer). delta: the sublayer's result,
    [n, width] of either dtype or [k, n, width] partial sums; then x_t <- sum_s mix[s, t] x_s + write[t] * delta_scale *
    delta (mix float32 [parts, parts] or None = identity; write float32 [parts] or None = ones). The norm reads u =
    sum_t read[t] x_t (None = ones): out[r] = (u - mean) / sqrt(var + eps) * weight + bias for row rows[r] or r. out None:
    only the update is made."""
    _cuda(streams, weight, bias, out, init, delta, mix, write, read, rows)
    width = weight.numel()
    if streams.dtype != torch.float32 or not streams.is_contiguous() or streams.shape[-1] != parts * width \
            or weight.dtype != torch.float32 or not 0 < parts <= STREAM_MAX_PARTS:
        raise InvalidArgument("stream_layer_norm: streams float32 contiguous [n, parts * width], weight float32 [width]")
    for t, n in ((bias, width), (mix, parts * parts), (write, parts), (read, parts)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise InvalidArgument("stream_layer_norm: bias, mix, write and read are float32 of width, parts^2, parts, parts")
    if init is not None and (init.dtype != torch.float32 or not init.is_contiguous() or init.shape[-1] != width):
        raise InvalidArgument("stream_layer_norm: init float32 contiguous [n, width]")
    total = streams.shape[0]
    if out is not None:
        if not out.is_contiguous() or out.shape[-1] != width:
            raise InvalidArgument("stream_layer_norm: out contiguous [rows, width]")
        n_out = out.shape[0]
    else:
        n_out = total if n_rows is None else n_rows
    if rows is not None and (rows.dtype != torch.int32 or rows.numel() < n_out):
        raise InvalidArgument("stream_layer_norm: rows must be int32 with one entry per output row")
    if rows is None and total < n_out:
        raise InvalidArgument("stream_layer_norm: fewer input rows than output rows")
    k, part_stride = _delta_parts(delta, width, "stream_layer_norm")
    out_code = dtype_code(out.dtype) if out is not None else 0
    dd = dtype_code(delta.dtype) if delta is not None else out_code
    check_limits("layer_norm", rows=total)
    _take_ahead()
    _check(_fn("layer_norm", "dl_stream_layer_norm")(
        out_code, dd, _p(streams), parts, width, _p(init), _p(delta), k, part_stride, delta_scale, _p(mix), _p(write),
        _p(read), _p(weight), _p(bias), eps, _p(out), _p(rows), n_out, total, _stream()), "stream_layer_norm")


def stream_sum(streams: torch.Tensor, parts: int, out: torch.Tensor, delta: Optional[torch.Tensor] = None,
               delta_scale: float = 1.0, mix: Optional[torch.Tensor] = None, write: Optional[torch.Tensor] = None) -> None:
    """out[n, width] (float32) = the sum of a stream's parts, after the pending update of stream_layer_norm (which is
    not written back)."""
    _cuda(streams, out, delta, mix, write)
    rows, width = out.shape
    if streams.dtype != torch.float32 or out.dtype != torch.float32 or not streams.is_contiguous() or not out.is_contiguous() \
            or streams.shape[-1] != parts * width or streams.shape[0] < rows:
        raise InvalidArgument("stream_sum: streams float32 [n, parts * width], out float32 [n, width]")
    k, part_stride = _delta_parts(delta, width, "stream_sum")
    _check(_fn("layer_norm", "dl_stream_sum")(dtype_code(delta.dtype) if delta is not None else 0, _p(streams), parts, width,
                                              _p(delta), k, part_stride, delta_scale, _p(mix), _p(write), _p(out), rows,
                                              _stream()), "stream_sum")


def gla_scan(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, z: torch.Tensor, tau: float, q_scale: float,
             state: torch.Tensor, q_start: torch.Tensor, state_slots: torch.Tensor, o: torch.Tensor, requests: int,
             heads: int, dim: int, vdim: int, z_bias: Optional[torch.Tensor] = None) -> None:
    """Gated linear attention over the rows of a step, request by request from and into its state row: per head
    S <- diag(sigmoid(z)^(1/tau)) S + k v^T, o = S^T (q * q_scale). proj holds q, k (heads * dim each) and v (heads *
    vdim) from the given columns; z: float32 [rows, heads * dim] (plus z_bias, float32 [heads * dim], when given), turned into the
    decays in place; state: float32 [slots, >= heads * vdim * dim], S kept
    transposed; o: float32 contiguous [rows, heads * vdim]. See csrc/gla.cu."""
    from .device import sm_count
    _cuda(proj, z, state, q_start, state_slots, o)
    _rows_contiguous(proj, "proj")
    _rows_contiguous(z, "z")
    rows = proj.shape[0]
    if z.dtype != torch.float32 or z.shape[0] < rows or z.shape[1] < heads * dim or o.dtype != torch.float32 \
            or not o.is_contiguous() or o.shape != (rows, heads * vdim):
        raise InvalidArgument("gla_scan: z float32 [rows, heads * dim], o float32 contiguous [rows, heads * vdim]")
    if max(q_col, k_col) + heads * dim > proj.shape[1] or v_col + heads * vdim > proj.shape[1]:
        raise InvalidArgument("gla_scan: q, k or v lie outside the projection")
    if dim > 512 or not tau > 0:
        raise Unsupported(f"gla_scan: a state of {dim} rows (512 at most), tau {tau} (positive)")
    _state_rows(state, heads * dim * vdim, "gla_scan")
    if z_bias is not None and (z_bias.dtype != torch.float32 or z_bias.numel() != heads * dim):
        raise InvalidArgument("gla_scan: z_bias float32 [heads * dim]")
    _cuda(z_bias)
    _check(_fn("gla", "dl_gla_decay")(_p(z), z.stride(0), rows, heads * dim, _p(z_bias), tau, _stream()), "gla_decay")
    _check(_fn("gla", "dl_gla_scan")(dtype_code(proj.dtype), _p(proj), proj.stride(0), q_col, k_col, v_col, _p(z), z.stride(0),
                                     q_scale, _p(state), state.stride(0), _p(q_start), _p(state_slots), _p(o), requests,
                                     heads, dim, vdim, sm_count(), _stream()), "gla_scan")


MOE_MAX_EXPERTS = 256
MOE_TILE_ROWS = 32          # places a tile of the kernels for few places an expert
MOE_WIDE_TILE_ROWS = 128    # of the wide tensor-core kernel
MOE_WIDE_FROM = int(os.environ.get("DYNALM_MOE_WIDE_FROM", "48"))     # places an expert on average from which tiles are wide
MOE_TENSOR_CORES = os.environ.get("DYNALM_MOE_TC", "1") != "0"


def moe_max_tiles(pairs: int, experts: int, tile_rows: int = MOE_TILE_ROWS) -> int:
    """The most row tiles the experts' products of a step can have (csrc/moe.cu)."""
    return pairs // tile_rows + min(experts, pairs)


def moe_tile_rows(pairs: int, experts: int, a: torch.Tensor, widths) -> int:
    """Places a tile for a step of `pairs` pairs: 128 where the wide tensor-core kernel applies (bfloat16, every inner
    size in `widths` a multiple of 64) and an expert gets enough places on average, else 32."""
    wide = (MOE_TENSOR_CORES and a.dtype == torch.bfloat16 and all(w % 64 == 0 for w in widths)
            and pairs >= MOE_WIDE_FROM * experts)
    return MOE_WIDE_TILE_ROWS if wide else MOE_TILE_ROWS


def moe_route(logits: torch.Tensor, top: int, groups: int, keep: int, scale: float, ids: torch.Tensor,
              weights: torch.Tensor) -> None:
    """Per row of float32 router logits [tokens, experts]: softmax over all experts, the `keep` best of `groups` equal
    groups of neighbouring experts (a group's score: its largest), the `top` best experts of those groups (ids int32
    [tokens, top]) and their scores over their sum, times `scale` (weights float32 [tokens, top])."""
    _cuda(logits, ids, weights)
    _rows_contiguous(logits, "logits")
    tokens, experts = logits.shape
    if logits.dtype != torch.float32 or ids.dtype != torch.int32 or weights.dtype != torch.float32 \
            or not ids.is_contiguous() or not weights.is_contiguous() or ids.numel() < tokens * top or weights.numel() < tokens * top:
        raise InvalidArgument("moe_route: logits float32, ids int32 [tokens, top], weights float32 [tokens, top]")
    if experts > MOE_MAX_EXPERTS or top > experts or groups <= 0 or experts % groups or not 0 < keep <= groups \
            or top > keep * (experts // groups):
        raise Unsupported(f"moe_route: {experts} experts in {groups} groups, {keep} kept, {top} a token")
    _check(_fn("moe", "dl_moe_route")(_p(logits), logits.stride(0), tokens, experts, top, groups, keep, scale, _p(ids),
                                      _p(weights), _stream()), "moe_route")


def moe_group(ids: torch.Tensor, pairs: int, experts: int, place_of: torch.Tensor, pair_at: torch.Tensor,
              tiles: torch.Tensor, n_tiles: torch.Tensor, tile_rows: int = MOE_TILE_ROWS) -> None:
    """The (token, expert) pairs of a step in the order of their experts: place_of[pair], pair_at[place] (int32, one per
    pair), and the row tiles of the experts' products, tiles[i] = (expert, first place, places <= tile_rows), n_tiles[0]
    of them."""
    _cuda(ids, place_of, pair_at, tiles, n_tiles)
    if any(t.dtype != torch.int32 or not t.is_contiguous() for t in (ids, place_of, pair_at, tiles, n_tiles)) \
            or min(ids.numel(), place_of.numel(), pair_at.numel()) < pairs or tiles.numel() < 3 * moe_max_tiles(pairs, experts, tile_rows):
        raise InvalidArgument("moe_group: int32 arrays of one entry per pair, tiles of three per possible tile")
    if experts > MOE_MAX_EXPERTS:
        raise Unsupported(f"moe_group: {experts} experts ({MOE_MAX_EXPERTS} at most)")
    _check(_fn("moe", "dl_moe_group")(_p(ids), pairs, experts, _p(place_of), _p(pair_at), _p(tiles), _p(n_tiles), tile_rows,
                                      _stream()), "moe_group")


def moe_linear(a: torch.Tensor, pair_at: Optional[torch.Tensor], top_div: int, w: torch.Tensor, c: torch.Tensor,
               tiles: torch.Tensor, n_tiles: torch.Tensor, max_tiles: int, act: str = "none",
               tile_rows: int = MOE_TILE_ROWS) -> None:
    """c[place] = act(a[row of place] w[expert of place]^T) for every place of every tile: w [experts, N, K], a rows of K
    numbers (the row of a place is pair_at[place] // top_div, or the place itself when pair_at is None), c [places, N]
    of a's dtype or float32. act: "none" or "relu2"."""
    _cuda(a, pair_at, w, c, tiles, n_tiles)
    _rows_contiguous(a, "a")
    _rows_contiguous(c, "c")
    if w.dim() != 3 or not w.is_contiguous() or w.dtype != a.dtype or a.shape[1] != w.shape[2] or c.shape[1] != w.shape[1] \
            or c.dtype not in (a.dtype, torch.float32) or act not in ("none", "relu2"):
        raise InvalidArgument("moe_linear: w [experts, N, K] of a's dtype, a [rows, K], c [places, N] of a's dtype or float32")
    _check(_fn("moe", "dl_moe_linear")(dtype_code(a.dtype), dtype_code(c.dtype), _p(a), a.stride(0), _p(pair_at), top_div,
                                       _p(w), w.shape[1], w.shape[2], _p(c), c.stride(0), _p(tiles), _p(n_tiles), max_tiles,
                                       1 if act == "relu2" else 0, 1 if MOE_TENSOR_CORES else 0, tile_rows, _stream()),
           "moe_linear")


def moe_combine(c: torch.Tensor, place_of: torch.Tensor, weights: torch.Tensor, top: int, y: torch.Tensor) -> None:
    """y[t] = sum_k weights[t, k] * c[place_of[t * top + k]] in float32, in the order of k. c: float32 [places, width]."""
    _cuda(c, place_of, weights, y)
    tokens, width = y.shape
    if c.dtype != torch.float32 or not c.is_contiguous() or c.shape[1] != width or not y.is_contiguous() \
            or place_of.dtype != torch.int32 or weights.dtype != torch.float32:
        raise InvalidArgument("moe_combine: c float32 [places, width], y contiguous [tokens, width]")
    _check(_fn("moe", "dl_moe_combine")(dtype_code(y.dtype), _p(c), width, _p(place_of), _p(weights), top, _p(y), tokens,
                                        _stream()), "moe_combine")


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    """x[r, :] += bias over the rows of x (float32 bias), in place."""
    _cuda(x, bias)
    _rows_contiguous(x, "x")
    if bias.dtype != torch.float32 or bias.numel() != x.shape[1]:
        raise InvalidArgument("add_bias: bias float32 [columns of x]")
    _check(_fn("gates", "dl_add_bias")(dtype_code(x.dtype), _p(x), x.stride(0), _p(bias), x.shape[0], x.shape[1], _stream()),
           "add_bias")


MASKED_FLASH_SIZES = {(d, d) for d in range(16, 129, 16)} | {(32, 16), (48, 32), (64, 32), (96, 48), (96, 64), (128, 64),
                                                             (64, 128), (32, 64), (48, 16), (16, 32)}


def masked_flash_attention(q: torch.Tensor, k_cache: torch.Tensor, k_row: int, v_cache: torch.Tensor, v_row: int,
                           block_table: torch.Tensor, q_tiles: torch.Tensor, n_tiles: int, out: torch.Tensor, n_heads: int,
                           n_kv_heads: int, key_dim: int, value_dim: int, page_size: int, scale: float, window: int = 0,
                           keep_first: int = 0, sink: bool = False, one_token_tiles: bool = False, parts: int = 1,
                           partial: Optional[torch.Tensor] = None) -> None:
    """Flash attention of query tiles over the paged cache, bfloat16, with keys of key_dim and values of value_dim
    numbers (a pair of MASKED_FLASH_SIZES), kept first tokens behind the window and an optional extra term exp(0) in the
    denominator; see csrc/attention_masked_flash.cu. q_tiles: int32 [n_tiles, 4] = (request, first row, rows <= 128,
    first position). k_cache / v_cache point at the first token's keys / values, k_row / v_row elements between tokens.
    one_token_tiles: every tile is a single token, tile i being row i of q (a decode step); the heads that share a KV head
    then share a block, and with parts > 1 a row's key tiles are dealt over that many blocks whose results a second
    kernel merges (partial: float32 scratch of masked_flash_partial_floats elements)."""
    _cuda(q, k_cache, v_cache, block_table, q_tiles, out)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise Unsupported("masked flash attention: bfloat16 only")
    if (key_dim, value_dim) not in MASKED_FLASH_SIZES or page_size & (page_size - 1) or n_heads % n_kv_heads:
        raise Unsupported(f"masked flash attention: keys of {key_dim} and values of {value_dim}, page size {page_size}, "
                          f"heads {n_heads}:{n_kv_heads}")
    if q.stride(0) % 8 or out.stride(0) % 2 or q.data_ptr() % 16 or out.data_ptr() % 4 or q_tiles.data_ptr() % 16 \
            or k_row % 8 or v_row % 8 or k_cache.data_ptr() % 16 or v_cache.data_ptr() % 16:
        raise Unsupported("masked flash attention: q and cache rows must be 16-byte aligned, out rows 4-byte aligned")
    if q_tiles.dtype != torch.int32 or q_tiles.numel() < 4 * n_tiles:
        raise InvalidArgument("masked flash attention: q_tiles must be int32 [n_tiles, 4]")
    if parts > 1 and (not one_token_tiles or partial is None or partial.dtype != torch.float32
                      or partial.numel() < masked_flash_partial_floats(n_tiles, n_heads, value_dim, parts) or n_tiles > q.shape[0]):
        raise InvalidArgument("masked flash attention: parts go with single-token tiles and a float32 scratch for them")
    _cuda(partial)
    check_limits("attention_masked_flash", pages=k_cache.shape[0], requests=block_table.shape[0], rows=q.shape[0])
    _check(_fn("attention_masked_flash", "dl_masked_flash_attention")(
        _p(q), q.stride(0), _p(k_cache), k_row, _p(v_cache), v_row, _p(block_table), block_table.stride(0), _p(q_tiles),
        n_tiles, _p(out), out.stride(0), n_heads, n_kv_heads, key_dim, value_dim, page_size, scale, window, int(keep_first),
        1 if sink else 0, 1 if one_token_tiles else 0, int(parts), _p(partial) if parts > 1 else None, _stream()),
        "masked_flash_attention")


MASKED_FLASH_MAX_PARTS = 8


def masked_flash_partial_floats(rows: int, n_heads: int, value_dim: int, parts: int) -> int:
    return rows * n_heads * parts * (value_dim + 2)


def masked_flash_parts(rows: int, blocks_a_row: int, keys: int) -> int:
    """Into how many parts a decode step deals a row's key tiles: enough blocks to cover the GPU about twice, a part at
    least four key tiles (256 keys), at most MASKED_FLASH_MAX_PARTS, a power of two (`keys`: the longest row's, already
    rounded so that the launch shape changes only now and then)."""
    from .device import sm_count
    want = -(-2 * sm_count() // max(1, rows * blocks_a_row))
    parts = 1
    while parts * 2 <= min(want, MASKED_FLASH_MAX_PARTS, keys // 256):
        parts *= 2
    return parts


MOE_TCGEN05 = os.environ.get("DYNALM_MOE_TCGEN05", "1") != "0"      # 0: the experts' products of long steps on mma.sync


def moe_gather(a: torch.Tensor, pair_at: torch.Tensor, top_div: int, out: torch.Tensor) -> None:
    """out[place] = a[pair_at[place] // top_div]: the rows of a step (bfloat16) in the order of their experts."""
    _cuda(a, pair_at, out)
    _rows_contiguous(a, "a")
    pairs, K = out.shape
    if a.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or not out.is_contiguous() or a.shape[1] != K \
            or pair_at.dtype != torch.int32 or pair_at.numel() < pairs:
        raise InvalidArgument("moe_gather: a [rows, K] and out [pairs, K] bfloat16, pair_at int32 [pairs]")
    _check(_fn("moe", "dl_moe_gather")(_p(a), a.stride(0), _p(pair_at), top_div, _p(out), pairs, K, _stream()), "moe_gather")


def moe_linear_tcgen05_applies(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor) -> bool:
    """Whether the grouped tcgen05 product takes these operands (bfloat16, aligned rows, an output it can store)."""
    n = w.shape[1]
    return (MOE_TCGEN05 and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and a.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and c.data_ptr() % 16 == 0 and c.stride(1) == 1
            and (n % 8 == 0 and c.stride(0) % 8 == 0 if c.dtype == torch.bfloat16 else n % 4 == 0 and c.stride(0) % 4 == 0))


def moe_linear_tcgen05(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, tiles: torch.Tensor, n_tiles: torch.Tensor,
                       max_tiles: int, act: str = "none") -> None:
    """c[place] = act(a[place] w[expert of place]^T) on the tcgen05 tensor cores: a [places, K] bfloat16 IN PLACE ORDER
    (moe_gather), w [experts, N, K], c [places, N] bfloat16 or float32 (act "none" only), tiles of at most 128 places as
    moe_group lists them with tile_rows = 128. See csrc/gemm_tcgen05.cu (dl_gemm_tcgen05_grouped)."""
    _cuda(a, w, c, tiles, n_tiles)
    if not moe_linear_tcgen05_applies(a, w, c) or w.dim() != 3 or a.shape[1] != w.shape[2] or c.shape != (a.shape[0], w.shape[1]) \
            or act not in ("none", "relu2") or (act == "relu2" and c.dtype != torch.bfloat16):
        raise Unsupported("moe_linear_tcgen05: bfloat16 operands with 16-byte aligned rows; relu2 with a bfloat16 result")
    mode = 4 if act == "relu2" else (0 if c.dtype == torch.bfloat16 else 1)
    status = _status_word(a.device)
    _check(_fn("gemm_tcgen05", "dl_gemm_tcgen05_grouped")(
        _p(a), a.stride(0), a.shape[0], _p(w), w.shape[0], w.shape[1], w.shape[2], _p(c), c.stride(0), mode, _p(tiles),
        _p(n_tiles), max_tiles, _p(status), _stream()), "moe_linear_tcgen05")
