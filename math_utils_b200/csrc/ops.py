"""Python face of the CUDA kernels: torch tensors in, launches on the current stream.

The kernels live in one shared object built from the ``.cu`` files beside this
module (``build.py``) and are called through their ``extern "C"`` launchers.
There is no other implementation behind these functions: if the library cannot
be built or loaded, or a tensor is not on a CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from . import build

ACT_CODES = {None: 0, "none": 0, "gelu_new": 1, "gelu": 2, "relu2": 4}      # relu2: max(z, 0)^2
GATE_ACT_CODES = {"gelu_new": 1, "gelu": 2, "silu": 3}       # what a gated feed-forward may put on its gate

_ERRORS = {
    1: "bad argument (a size, stride or pointer the kernel cannot take)",
    2: "unsupported size for this kernel",
    3: "the CUDA runtime refused the launch",
    4: "a pointer or stride breaks an alignment rule of this kernel",
    5: "the kernel library could not set itself up on this device",
}


class KernelError(RuntimeError):
    pass


_lib = None
_lock = threading.Lock()


def _switch(name: str) -> bool:
    return os.environ.get(name, "1") != "0"


# Switches for measurements, read once when this module is imported:
#   MU_B200_PDL=0         plain stream order between kernels (no programmatic dependent launch)
#   MU_B200_ATT_TC=0      single-token attention on CUDA cores instead of mma.sync
#   MU_B200_PREFILL_TC=0  prompt attention on mma.sync instead of tcgen05
#   MU_B200_LATENT_TC=0   latent attention and the experts' products on CUDA cores instead of mma.sync
PDL, ATT_TC, PREFILL_TC = _switch("MU_B200_PDL"), _switch("MU_B200_ATT_TC"), _switch("MU_B200_PREFILL_TC")
LATENT_TC = _switch("MU_B200_LATENT_TC")
MAPPED_TC = _switch("MU_B200_MAPPED_TC")     # =0: prompt attention with score maps on CUDA cores instead of mma.sync

_c_int, _c_ll, _c_f, _c_p, _c_ull = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p, ctypes.c_ulonglong

_SIGNATURES = {
    "mu_copy_async": [_c_p, _c_p, _c_ll, _c_p],
    "mu_embed": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_f, _c_p],
    "mu_layernorm": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_f, _c_int, _c_p],
    "mu_gemm_simt": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll,
                     _c_int, _c_int, _c_int, _c_p],
    "mu_gemm_skinny": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll,
                       _c_int, _c_int, _c_p],
    "mu_gemm_tc_split_workspace": [_c_p, _c_ll, _c_p, _c_int],
    "mu_gemm_tc": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll,
                   _c_int, _c_int, _c_int, _c_int, _c_p, _c_p],
    "mu_gemm_rows": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll,
                     _c_int, _c_int, _c_int, _c_p, _c_p],
    "mu_kv_append": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
                     _c_int, _c_p, _c_int, _c_p, _c_int, _c_p],
    "mu_attention": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_p, _c_p, _c_int,
                     _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _c_p, _c_p, _c_int, _c_p],
    "mu_attention_prefill": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_p, _c_p, _c_p, _c_int,
                             _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_p],
    "mu_attention_prefill_tc": [_c_p, _c_ll, _c_int, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_int, _c_int, _c_p, _c_p,
                                _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_ll, _c_p, _c_ll,
                                _c_p, _c_int, _c_p, _c_p],
    "mu_layernorm_gemm_tc": [_c_p, _c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int,
                             _c_ll, _c_ll, _c_ll, _c_int, _c_int, _c_p, _c_p],
    "mu_argmax": [_c_p, _c_ll, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p],
    "mu_gemm_stream_fits": [_c_int, _c_int, _c_ll, _c_int],
    "mu_gemm_stream": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int,
                       _c_ll, _c_ll, _c_int, _c_int, _c_p, _c_p],
    "mu_gemm_skinny_ln": [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int,
                          _c_ll, _c_ll, _c_ll, _c_int, _c_int, _c_p],
    "mu_attention_decode": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_int, _c_int,
                            _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _c_int, _c_p],
    "mu_attention_decode_tc": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_int, _c_int,
                               _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_p, _c_p],
    "mu_embed_pair": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_ll,
                      _c_ll, _c_int, _c_int, _c_p],
    "mu_rms_norm_out": [_c_p, _c_ll, _c_p, _c_ll, _c_f, _c_f, _c_p, _c_p, _c_f, _c_f, _c_f, _c_p, _c_ll, _c_int, _c_int,
                        _c_p, _c_ll, _c_int, _c_int, _c_p],
    "mu_gated_act": [_c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p],
    "mu_scaled_sum": [_c_p, _c_ll, _c_f, _c_p, _c_ll, _c_f, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p],
    "mu_cast_rows": [_c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_p],
    "mu_qk_prepare": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_f, _c_int, _c_f, _c_int, _c_int, _c_int,
                      _c_int, _c_int, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p, _c_int, _c_p, _c_int],
    "mu_mapped_attention": [_c_p, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                            _c_int, _c_f, _c_int, _c_f, _c_f, _c_f, _c_int, _c_p, _c_ll, _c_int, _c_p,
                            _c_p, _c_int, _c_p, _c_ll, _c_int],
    "mu_mapped_decode_fits": [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int],
    "mu_mapped_decode_scratch": [_c_int, _c_int, _c_int, _c_int],
    "mu_mapped_attention_decode": [_c_p, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                                   _c_int, _c_f, _c_int, _c_f, _c_f, _c_f, _c_int, _c_p, _c_p, _c_ll, _c_int, _c_p,
                                   _c_p, _c_int, _c_p, _c_ll, _c_int],
    "mu_mapped_attention_mma_fits": [_c_int, _c_int, _c_int, _c_int, _c_int],
    "mu_mapped_attention_mma": [_c_p, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
                                _c_int, _c_int, _c_f, _c_int, _c_f, _c_f, _c_f, _c_int, _c_p, _c_ll, _c_p,
                                _c_p, _c_int, _c_p, _c_ll, _c_int],
    "mu_qkv_norm_rows": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_f, _c_int, _c_int, _c_int, _c_int, _c_int,
                         _c_int, _c_p, _c_int, _c_f, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p, _c_int, _c_p],
    "mu_residual_add_norm": [_c_p, _c_ll, _c_p, _c_ll, _c_f, _c_p, _c_f, _c_int, _c_int, _c_p, _c_ll, _c_int, _c_p],
    "mu_delta_prepare": [_c_p, _c_int, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f,
                         _c_p, _c_p, _c_p, _c_int, _c_p],
    "mu_delta_scan_max_dk": [],
    "mu_delta_scan": [_c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p, _c_p, _c_ll,
                      _c_ll, _c_p, _c_int, _c_p],
    "mu_xielu": [_c_p, _c_ll, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p],
    "mu_ssd_conv": [_c_p, _c_ll, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_ll,
                    _c_int, _c_p, _c_p],
    "mu_ssd_scan": [_c_p, _c_int, _c_p, _c_ll, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p,
                    _c_p, _c_p, _c_ll, _c_ll, _c_p, _c_int, _c_p],
    "mu_gated_group_norm": [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_int, _c_int, _c_int, _c_f, _c_p, _c_ll, _c_int, _c_p, _c_int],
    "mu_dynamic_tanh": [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p],
    "mu_rms_norm": [_c_p, _c_ll, _c_int, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_f, _c_p],
    "mu_sigmoid_gate": [_c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p],
    "mu_rotary": [_c_p, _c_ll, _c_int, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_p, _c_p, _c_f, _c_int, _c_int, _c_int,
                  _c_int, _c_p],
    "mu_latent_append": [_c_p, _c_ll, _c_p, _c_f, _c_p, _c_f, _c_int, _c_int, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int,
                         _c_int, _c_p, _c_int, _c_p, _c_ll, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_p, _c_int],
    "mu_moe_combine_tanh": [_c_p, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_p],
    "mu_latent_attention": [_c_p, _c_p, _c_p, _c_int, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int,
                            _c_p, _c_ll, _c_p, _c_p, _c_int, _c_p, _c_p],
    "mu_latent_merge": [_c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p, _c_ll, _c_int, _c_p, _c_p],
    "mu_latent_attention_mma_fits": [_c_int, _c_int, _c_int],
    "mu_latent_attention_mma": [_c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_f,
                                _c_int, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_int],
    "mu_moe_route": [_c_p, _c_ll, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_p, _c_p,
                     _c_p, _c_f, _c_p, _c_p],
    "mu_moe_group": [_c_p, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int],
    "mu_moe_gemm": [_c_p, _c_ll, _c_p, _c_int, _c_p, _c_p, _c_ll, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p, _c_ll,
                    _c_int, _c_int, _c_p, _c_int],
    "mu_moe_gemm_mma": [_c_p, _c_ll, _c_p, _c_int, _c_p, _c_p, _c_ll, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p,
                        _c_ll, _c_int, _c_p, _c_int],
    "mu_heads_gemm": [_c_p, _c_ll, _c_ll, _c_p, _c_ll, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p, _c_ll, _c_ll, _c_int,
                      _c_p, _c_ll, _c_p],
    "mu_moe_combine": [_c_p, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p, _c_ll, _c_p, _c_p, _c_ll, _c_int, _c_p,
                       _c_ll, _c_p, _c_int],
    "mu_rms_norm_pair": [_c_p, _c_ll, _c_p, _c_p, _c_f, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p],
    "mu_softcap": [_c_p, _c_ll, _c_int, _c_int, _c_f, _c_p],
    "mu_moe_tile_rows": [],
    "mu_sample": [_c_p, _c_ll, _c_int, _c_int, _c_f, _c_int, _c_ull, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int,
                  _c_p, _c_p, _c_p],
}


def library() -> ctypes.CDLL:
    """The loaded kernel library; builds it at the first call if needed."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build.library_path()
                try:
                    lib = ctypes.CDLL(path)
                except OSError as e:
                    raise KernelError(f"cannot load the CUDA kernels of math_utils_b200 from {path}: {e}") from None
                for name, argtypes in _SIGNATURES.items():
                    try:
                        fn = getattr(lib, name)
                    except AttributeError:
                        continue          # optional kernels are looked up where they are used
                    fn.argtypes = argtypes
                    fn.restype = _c_int
                if not PDL:
                    lib.mu_set_pdl(0)         # plain stream order between kernels
                _lib = lib
    return _lib


launch_count = 0      # kernels of this library launched so far (a merge after a split counts too)


def _check(code: int, what, launches: int = 1) -> None:
    """``what`` names the call for the error message: a string, or a tuple of a
    format and its arguments, put together only when there is an error."""
    global launch_count
    if code != 0:
        if isinstance(what, tuple):
            what = what[0].format(*what[1:])
        raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")
    launch_count += launches


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream        # the current stream's handle without a Stream object
except AttributeError:                                       # pragma: no cover
    _raw_stream = None


_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("math_utils_b200 kernels run on CUDA tensors only; got a tensor on " + str(t.device))


def _is_bf16(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise KernelError(f"kernels take bfloat16 or float32, got {t.dtype}")


def _i32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{name} must be a contiguous int32 tensor")


def set_pdl(enabled: bool) -> None:
    """Switches programmatic stream serialization of the launches on or off
    (on unless MU_B200_PDL=0 when the module was imported): with it a kernel may start, and fetch what no
    kernel of the step writes, while the kernel before it ends.  Launches
    already recorded in a CUDA graph keep the mode they were recorded with."""
    library().mu_set_pdl(1 if enabled else 0)


def copy_async(dst: torch.Tensor, src: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> None:
    """dst <- src (same size and dtype, contiguous; host tensors pinned) as a
    plain asynchronous copy on the current stream, or on ``stream``.  The
    caller keeps both tensors alive until the copy is over (a copy recorded in
    a CUDA graph: as long as the graph)."""
    if dst.dtype != src.dtype or dst.numel() != src.numel() or not dst.is_contiguous() or not src.is_contiguous():
        raise KernelError("copy_async needs contiguous tensors of one dtype and size")
    for t in (dst, src):
        if not t.is_cuda and not t.is_pinned():
            raise KernelError("copy_async needs pinned host memory")
    _check(library().mu_copy_async(dst.data_ptr(), src.data_ptr(), dst.numel() * dst.element_size(),
                                   _stream() if stream is None else stream.cuda_stream), "copy_async", launches=0)


_workspaces = {}
_retired = []


def zeroed_workspace(name: str, device, n_bytes: int) -> torch.Tensor:
    """A device buffer that kernels with tickets use and leave zero again.  It
    is kept per purpose and device and only ever grows, so its address stays put
    for launches recorded in a CUDA graph as long as no larger size is asked for
    later."""
    key = (name, str(device))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < n_bytes:
        if buf is not None:
            _retired.append(buf)        # a recorded graph may still point at it
        buf = torch.zeros(max(n_bytes, 65536), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


# ------------------------------------------------------------------ elementwise
def embed(ids: torch.Tensor, positions: Optional[torch.Tensor], table: torch.Tensor,
          pos_table: Optional[torch.Tensor], out: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """out[t] = table[ids[t]] * scale + pos_table[positions[t]] as float32 [T, hidden]."""
    _need_cuda(ids, positions, table, pos_table)
    _i32(ids, "ids"); _i32(positions, "positions")
    n, hidden = ids.numel(), table.shape[1]
    if pos_table is not None and (pos_table.dtype != table.dtype or pos_table.shape[1] != hidden):
        raise KernelError("the position table must match the token table in dtype and width")
    if not table.is_contiguous() or (pos_table is not None and not pos_table.is_contiguous()):
        raise KernelError("embedding tables must be contiguous")
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _check(library().mu_embed(_ptr(ids), _ptr(positions),
                              _ptr(table), _ptr(pos_table), _ptr(out), n, hidden, _is_bf16(table), float(scale),
                              _stream()),
           "embed")
    return out


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float,
              out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LayerNorm of float32 rows (optionally the rows that ``rows`` picks)."""
    _need_cuda(x, gamma, beta, rows)
    _i32(rows, "rows")
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("layernorm input must be contiguous float32")
    if gamma.dtype != torch.float32 or (beta is not None and beta.dtype != torch.float32):
        raise KernelError("layernorm parameters must be float32")
    hidden = x.shape[-1]
    n = rows.numel() if rows is not None else x.numel() // hidden
    if out is None:
        out = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
    _check(library().mu_layernorm(_ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out), n, hidden,
                                  float(eps), _is_bf16(out), _stream()), ("layernorm(hidden={})", hidden))
    return out


def dynamic_tanh(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], alpha: torch.Tensor,
                 out_dtype: Optional[torch.dtype] = None, rows: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, add: bool = False) -> torch.Tensor:
    """tanh(alpha x) * weight + bias of float32 rows (optionally the rows that ``rows`` picks); ``alpha`` is a
    float32 scalar on the device.  With ``add`` the result is added to the float32 ``out``."""
    _need_cuda(x, weight, bias, alpha, rows, out)
    _i32(rows, "rows")
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("dynamic_tanh input must be float32 [rows, hidden] with unit inner stride")
    for t in (weight, bias, alpha):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError("dynamic_tanh parameters must be contiguous float32")
    hidden = x.shape[1]
    n = rows.numel() if rows is not None else x.shape[0]
    if out is None:
        if add:
            raise KernelError("dynamic_tanh(add=True) needs the tensor to add to")
        out = torch.empty((n, hidden), dtype=out_dtype or torch.float32, device=x.device)
    if out.shape != (n, hidden) or out.stride(1) != 1 or (add and out.dtype != torch.float32):
        raise KernelError("dynamic_tanh output has the wrong shape, stride or dtype")
    _check(library().mu_dynamic_tanh(_ptr(x), x.stride(0), _ptr(rows), _ptr(weight), _ptr(bias), _ptr(alpha), _ptr(out),
                                     out.stride(0), n, hidden, _is_bf16(out), int(add), _stream()),
           ("dynamic_tanh(hidden={})", hidden))
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: Optional[torch.dtype] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over each row ([rows, n] views with unit inner stride, bfloat16 or
    float32); statistics in float32."""
    _need_cuda(x, weight, out)
    if x.dim() != 2 or x.stride(1) != 1 or weight.dtype != torch.float32 or weight.numel() != x.shape[1]:
        raise KernelError("rms_norm takes [rows, n] with unit inner stride and a float32 weight of n values")
    if out is None:
        out = torch.empty(tuple(x.shape), dtype=out_dtype or x.dtype, device=x.device)
    if out.shape != x.shape or out.stride(1) != 1:
        raise KernelError("rms_norm output has the wrong shape or stride")
    _check(library().mu_rms_norm(_ptr(x), x.stride(0), _is_bf16(x), _ptr(weight), _ptr(out), out.stride(0), _is_bf16(out),
                                 x.shape[0], x.shape[1], float(eps), _stream()), ("rms_norm(n={})", x.shape[1]))
    return out


def rms_norm_out(x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float = 0.0, scale: float = 1.0,
                 out_dtype: Optional[torch.dtype] = None, rows: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, add: bool = False,
                 copy: Optional[torch.Tensor] = None, second=None) -> torch.Tensor:
    """scale * v / sqrt(mean(v^2) + eps) * (offset + weight) of float32 rows v = x (optionally the rows that ``rows``
    picks), written to ``out`` or, with ``add``, added to the float32 ``out``.  ``copy`` (bfloat16, shaped like
    ``out``) receives what ``out`` then holds.  ``second`` = (a, x2, b): the rows are v = a * x + b * x2."""
    a, x2, b = second if second is not None else (1.0, None, 0.0)
    _need_cuda(x, weight, rows, out, copy, x2)
    if x2 is not None and (x2.dtype != torch.float32 or x2.shape != x.shape or x2.stride(1) != 1):
        raise KernelError("rms_norm_out: the second input is float32 and shaped like the first")
    _i32(rows, "rows")
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("rms_norm_out input must be float32 [rows, n] with unit inner stride")
    if weight.dtype != torch.float32 or not weight.is_contiguous() or weight.numel() != x.shape[1]:
        raise KernelError("rms_norm_out takes a contiguous float32 weight of n values")
    n = x.shape[1]
    n_rows = rows.numel() if rows is not None else x.shape[0]
    if out is None:
        if add:
            raise KernelError("rms_norm_out(add=True) needs the tensor to add to")
        out = torch.empty((n_rows, n), dtype=out_dtype or torch.float32, device=x.device)
    if out.shape != (n_rows, n) or out.stride(1) != 1 or (add and out.dtype != torch.float32):
        raise KernelError("rms_norm_out output has the wrong shape, stride or dtype")
    if copy is not None and (copy.dtype != torch.bfloat16 or copy.shape != out.shape or copy.stride(1) != 1):
        raise KernelError("rms_norm_out: the copy is bfloat16 and shaped like the output")
    _check(library().mu_rms_norm_out(_ptr(x), x.stride(0), _ptr(x2), x2.stride(0) if x2 is not None else 0, float(a),
                                     float(b), _ptr(rows), _ptr(weight), float(offset), float(scale),
                                     float(eps), _ptr(out), out.stride(0), _is_bf16(out), int(add), _ptr(copy),
                                     copy.stride(0) if copy is not None else 0, n_rows, n, _stream()),
           ("rms_norm_out(n={})", n))
    return out


def cast_rows(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 rows [rows, n] as bfloat16."""
    _need_cuda(x, out)
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("cast_rows takes float32 [rows, n] with unit inner stride")
    if out is None:
        out = torch.empty(tuple(x.shape), dtype=torch.bfloat16, device=x.device)
    if out.dtype != torch.bfloat16 or out.shape != x.shape or out.stride(1) != 1:
        raise KernelError("cast_rows output must be bfloat16 of the input's shape")
    _check(library().mu_cast_rows(_ptr(x), x.stride(0), _ptr(out), out.stride(0), x.shape[0], x.shape[1], _stream()),
           "cast_rows")
    return out


def gated_act(a: torch.Tensor, out: torch.Tensor, act: str) -> torch.Tensor:
    """out[:, f] = act(a[:, f]) * a[:, F + f] for a [rows, 2F] (gate | up) and out [rows, F] of one dtype."""
    _need_cuda(a, out)
    if (a.dim() != 2 or out.dim() != 2 or a.shape[1] != 2 * out.shape[1] or a.shape[0] != out.shape[0]
            or a.dtype != out.dtype or a.stride(1) != 1 or out.stride(1) != 1):
        raise KernelError("gated_act takes [rows, 2F] and [rows, F] of one dtype with unit inner stride")
    if act not in GATE_ACT_CODES:
        raise KernelError(f"gated_act: no activation '{act}'; known: {', '.join(GATE_ACT_CODES)}")
    _check(library().mu_gated_act(_ptr(a), a.stride(0), _ptr(out), out.stride(0), out.shape[0], out.shape[1],
                                  GATE_ACT_CODES[act], _is_bf16(a), _stream()), "gated_act")
    return out


def scaled_sum(p: torch.Tensor, a: float, q: torch.Tensor, b: float, out: torch.Tensor, add: bool = False) -> torch.Tensor:
    """out (+)= a * p + b * q, all float32 [rows, n]."""
    _need_cuda(p, q, out)
    for t in (p, q, out):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or t.shape != out.shape:
            raise KernelError("scaled_sum takes float32 [rows, n] tensors of one shape with unit inner stride")
    _check(library().mu_scaled_sum(_ptr(p), p.stride(0), float(a), _ptr(q), q.stride(0), float(b), _ptr(out),
                                   out.stride(0), out.shape[0], out.shape[1], int(add), _stream()), "scaled_sum")
    return out


def embed_pair(ids: torch.Tensor, positions: torch.Tensor, tok_seq: torch.Tensor, seq_first: torch.Tensor,
               seq_slots: torch.Tensor, last_token: torch.Tensor, table: torch.Tensor, pair_table: torch.Tensor,
               mul_prev: int, mul_cur: int, single_tokens: bool, out: Optional[torch.Tensor] = None,
               copy: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = table[ids[t]] + pair_table[(previous * mul_prev + ids[t] * mul_cur) mod buckets] as float32, with
    buckets = pair_table's rows - 1 and that last row for a sequence's first token.  The token before the step's
    first token of a sequence is ``last_token[slot]``, which is then set to the sequence's last token of the step.
    ``copy`` (contiguous bfloat16 [T, hidden]) receives the same rows rounded."""
    _need_cuda(ids, positions, tok_seq, seq_first, seq_slots, last_token, table, pair_table, out, copy)
    if copy is not None and (copy.dtype != torch.bfloat16 or not copy.is_contiguous()
                             or tuple(copy.shape) != (ids.numel(), table.shape[1])):
        raise KernelError("embed_pair: the copy is contiguous bfloat16 [T, hidden]")
    for t, name in ((ids, "ids"), (positions, "positions"), (tok_seq, "tok_seq"), (seq_first, "seq_first"),
                    (seq_slots, "seq_slots"), (last_token, "last_token")):
        _i32(t, name)
    n, hidden = ids.numel(), table.shape[1]
    if (pair_table.dtype != table.dtype or pair_table.shape[1] != hidden or not table.is_contiguous()
            or not pair_table.is_contiguous() or pair_table.shape[0] < 2):
        raise KernelError("the pair table must match the token table in dtype and width")
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _check(library().mu_embed_pair(_ptr(ids), _ptr(positions), _ptr(tok_seq), _ptr(seq_first), _ptr(seq_slots),
                                   _ptr(last_token), _ptr(table), _ptr(pair_table), _ptr(out), _ptr(copy), n, seq_slots.numel(),
                                   hidden, pair_table.shape[0] - 1, int(mul_prev), int(mul_cur), _is_bf16(table),
                                   int(single_tokens), _stream()), "embed_pair", launches=1 if single_tokens else 2)
    return out


# ------------------------------------------------------------------ attention over cached rows with score maps
def qk_prepare(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], q_weight: Optional[torch.Tensor],
               k_weight: Optional[torch.Tensor], freqs: torch.Tensor, magnitude: float, rot_dims: int, eps: float,
               n_heads: int, n_kv_heads: int, maps: int, dim: int, vdim: int, tok_pos, tok_seq,
               block_table: Optional[torch.Tensor], page_tokens: int, rows: Optional[torch.Tensor],
               pairs: bool = False) -> None:
    """Unit rms times a weight, then the rotation, for every (head, map) slice of the queries (in place) and of the
    keys (into the token's cache row, with the values behind them).  ``k`` and ``v`` None: queries only.
    Without weights (both None) the slices are not normed.  ``pairs``: entry 2i turns with entry 2i + 1 instead of
    entry i with entry i + rot_dims / 2."""
    _need_cuda(q, k, v, q_weight, k_weight, freqs, tok_pos, tok_seq, block_table, rows)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        _i32(t, name)
    if q.stride(1) != 1 or q.shape[1] != n_heads * maps * dim:
        raise KernelError("qk_prepare: queries are [T, heads * maps * dim] with unit inner stride")
    if k is not None:
        if (k.dtype != q.dtype or v.dtype != q.dtype or rows.dtype != q.dtype or k.stride(1) != 1 or v.stride(1) != 1
                or k.shape[1] != n_kv_heads * maps * dim or v.shape[1] != n_kv_heads * vdim or not rows.is_contiguous()
                or rows.shape[1] != page_tokens or rows.shape[2] != n_kv_heads * (maps * dim + vdim)):
            raise KernelError("qk_prepare: keys, values and cache rows do not fit the sizes given")
    for w in (q_weight, k_weight, freqs):
        if w is not None and (w.dtype != torch.float32 or not w.is_contiguous()):
            raise KernelError("qk_prepare: weights and frequencies are contiguous float32")
    _check(library().mu_qk_prepare(_ptr(q), q.stride(0), _ptr(k), k.stride(0) if k is not None else 0, _ptr(v),
                                   v.stride(0) if v is not None else 0, _ptr(q_weight), _ptr(k_weight), _ptr(freqs),
                                   float(magnitude), int(rot_dims), float(eps), q.shape[0], int(n_heads),
                                   int(n_kv_heads), int(maps), int(dim), int(vdim), _ptr(tok_pos), _ptr(tok_seq),
                                   _ptr(block_table), block_table.shape[1] if block_table is not None else 0,
                                   int(page_tokens), _ptr(rows), _is_bf16(q), _stream(), int(pairs)),
           ("qk_prepare(dim={}, maps={})", dim, maps))


def mapped_attention(q: torch.Tensor, rows: torch.Tensor, block_table: torch.Tensor, page_tokens: int, tok_pos, tok_seq,
                     n_heads: int, n_kv_heads: int, maps: int, dim: int, vdim: int, scale: float, window: int,
                     out: torch.Tensor, lam: float = 0.0, out_scale: float = 1.0, eps: float = 0.0,
                     unit_rms: bool = False, tiles: Optional[torch.Tensor] = None,
                     tensor_cores: Optional[bool] = None, single_tokens: bool = False,
                     head_scale: Optional[torch.Tensor] = None, sink: bool = False,
                     gate: Optional[torch.Tensor] = None, chunk: int = 0) -> torch.Tensor:
    """Softmax attention of every (token, head) over the cached rows it sees (``window`` 0: all up to its own
    position), one result per score map over the same values; with two maps a1 - lam * a2.  ``unit_rms`` brings
    each head's result to unit rms (eps inside the root); ``out_scale`` multiplies it.

    ``tiles`` (int32 [n, 2]: first flat token and count <= 64 of runs of tokens of one sequence, as a prompt step
    has them) sends bfloat16 steps at the sizes ``mu_mapped_attention_mma`` takes to the tensor cores, unless
    ``tensor_cores`` is false.  ``single_tokens`` (every token is the one token of its sequence) takes the kernel
    that shares a sequence's pages out over blocks and lets the query heads of a kv head read them together.

    ``head_scale`` (float32, one per head) multiplies the head's scores besides ``scale``; ``sink`` adds to the
    softmax's denominator one key of score zero that has no value; ``gate`` ([T, heads] view in the compute dtype)
    multiplies each head's result by sigmoid(gate[t, h]); ``chunk`` c > 0 replaces the window: position p sees
    p - p % c .. p."""
    _need_cuda(q, rows, block_table, tok_pos, tok_seq, out, head_scale, gate)
    if head_scale is not None and (head_scale.dtype != torch.float32 or head_scale.numel() != n_heads
                                   or not head_scale.is_contiguous()):
        raise KernelError("mapped_attention: head_scale is one contiguous float32 per head")
    if gate is not None and (gate.dtype != rows.dtype or gate.dim() != 2 or gate.shape != (q.shape[0], n_heads)
                             or gate.stride(1) != 1):
        raise KernelError("mapped_attention: the gate is [T, heads] in the compute dtype with unit inner stride")
    extras = (_ptr(head_scale), int(sink), _ptr(gate), gate.stride(0) if gate is not None else 0, int(chunk))
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        _i32(t, name)
    if (q.dtype != rows.dtype or out.dtype != rows.dtype or q.stride(1) != 1 or out.stride(1) != 1
            or not rows.is_contiguous() or rows.shape[2] != n_kv_heads * (maps * dim + vdim)
            or q.shape[1] != n_heads * maps * dim or out.shape[1] != n_heads * vdim):
        raise KernelError("mapped_attention: queries, rows and output do not fit the sizes given")
    if single_tokens and library().mu_mapped_decode_fits(int(n_heads), int(n_kv_heads), int(maps), int(dim), int(vdim),
                                                         int(page_tokens), _is_bf16(rows)):
        lib = library()
        lib.mu_mapped_decode_scratch.restype = _c_ll
        need = int(lib.mu_mapped_decode_scratch(q.shape[0], int(n_heads), int(maps), int(vdim)))
        room = scratch("mapped_decode", q.device, need, torch.float32)
        _check(lib.mu_mapped_attention_decode(
            _ptr(q), q.stride(0), _ptr(rows), _ptr(block_table), block_table.shape[1], int(page_tokens), _ptr(tok_pos),
            _ptr(tok_seq), q.shape[0], int(n_heads), int(n_kv_heads), int(maps), int(dim), int(vdim), float(scale),
            int(window), float(lam), float(out_scale), float(eps), int(unit_rms), _ptr(room), _ptr(out), out.stride(0),
            _is_bf16(rows), _stream(), *extras),
            ("mapped_attention_decode(heads={}/{}, maps={}, dim={}, vdim={})", n_heads, n_kv_heads, maps, dim, vdim), launches=2)
        return out
    if tensor_cores is None:
        tensor_cores = MAPPED_TC
    if (tensor_cores and tiles is not None and rows.dtype == torch.bfloat16 and q.stride(0) % 8 == 0
            and out.stride(0) % 2 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 4 == 0
            and library().mu_mapped_attention_mma_fits(int(n_kv_heads), int(maps), int(dim), int(vdim), int(page_tokens))):
        _need_cuda(tiles)
        _i32(tiles, "tiles")
        _check(library().mu_mapped_attention_mma(
            _ptr(q), q.stride(0), _ptr(rows), _ptr(block_table), block_table.shape[1], int(page_tokens), _ptr(tok_pos),
            _ptr(tok_seq), _ptr(tiles), tiles.shape[0], int(n_heads), int(n_kv_heads), int(maps), int(dim), int(vdim),
            float(scale), int(window), float(lam), float(out_scale), float(eps), int(unit_rms), _ptr(out), out.stride(0),
            _stream(), *extras), ("mapped_attention_mma(heads={}/{}, maps={}, dim={}, vdim={})", n_heads, n_kv_heads, maps, dim, vdim))
        return out
    _check(library().mu_mapped_attention(_ptr(q), q.stride(0), _ptr(rows), _ptr(block_table), block_table.shape[1],
                                         int(page_tokens), _ptr(tok_pos), _ptr(tok_seq), q.shape[0], int(n_heads),
                                         int(n_kv_heads), int(maps), int(dim), int(vdim), float(scale), int(window),
                                         float(lam), float(out_scale), float(eps), int(unit_rms), _ptr(out),
                                         out.stride(0), _is_bf16(rows), _stream(), *extras),
           ("mapped_attention(heads={}/{}, maps={}, dim={}, vdim={})", n_heads, n_kv_heads, maps, dim, vdim))
    return out


# ------------------------------------------------------------------ state-space mixer
def ssd_conv(u: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], tok_seq, seq_first, seq_slots,
             state: torch.Tensor, single_tokens: bool, out: torch.Tensor) -> torch.Tensor:
    """silu of the short causal convolution of the channels ``u`` [T, channels] per sequence, float32 ``out``; the
    inputs before a sequence's first token of the step come from the head of ``state[slot]``, which is moved on."""
    _need_cuda(u, weight, bias, tok_seq, seq_first, seq_slots, state, out)
    for t, name in ((tok_seq, "tok_seq"), (seq_first, "seq_first"), (seq_slots, "seq_slots")):
        _i32(t, name)
    channels, taps = weight.shape
    if (u.stride(1) != 1 or u.shape[1] != channels or weight.dtype != torch.float32 or not weight.is_contiguous()
            or out.dtype != torch.float32 or not out.is_contiguous() or out.shape != (u.shape[0], channels)
            or state.dtype != torch.float32 or state.stride(1) != 1 or state.shape[1] < (taps - 1) * channels):
        raise KernelError("ssd_conv: inputs, weight, state or output do not fit")
    _check(library().mu_ssd_conv(_ptr(u), u.stride(0), _is_bf16(u), _ptr(weight), _ptr(bias), channels, taps, u.shape[0],
                                 seq_slots.numel(), _ptr(tok_seq), _ptr(seq_first), _ptr(seq_slots), _ptr(state),
                                 state.stride(0), int(single_tokens), _ptr(out), _stream()), "ssd_conv",
           launches=1 if single_tokens or taps == 1 else 2)
    return out


def ssd_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias, a_log, skip, n_heads: int, head_dim: int, n_state: int,
             groups: int, seq_first, seq_slots, state: torch.Tensor, state_offset: int, out: torch.Tensor) -> torch.Tensor:
    """The recurrence S = exp(-exp(A) dt) S + dt B x^T, y = S^T C + D x per (sequence, head) over the step's tokens,
    from and to ``state[slot][state_offset:]``; ``xbc`` [T, heads * P + 2 * groups * N] float32 = x | B | C."""
    _need_cuda(xbc, dt_raw, dt_bias, a_log, skip, seq_first, seq_slots, state, out)
    inner = n_heads * head_dim
    if (xbc.dtype != torch.float32 or not xbc.is_contiguous() or xbc.shape[1] != inner + 2 * groups * n_state
            or dt_raw.stride(1) != 1 or dt_raw.shape[1] != n_heads or out.dtype != torch.float32
            or not out.is_contiguous() or out.shape != (xbc.shape[0], inner) or state.dtype != torch.float32
            or state.shape[1] < state_offset + inner * n_state):
        raise KernelError("ssd_scan: inputs, state or output do not fit")
    for t in (dt_bias, a_log, skip):
        if t.dtype != torch.float32 or t.numel() != n_heads or not t.is_contiguous():
            raise KernelError("ssd_scan: one float32 per head for dt_bias, A_log and D")
    _check(library().mu_ssd_scan(_ptr(xbc), xbc.shape[1], _ptr(dt_raw), dt_raw.stride(0), _is_bf16(dt_raw), _ptr(dt_bias),
                                 _ptr(a_log), _ptr(skip), seq_slots.numel(), int(n_heads), int(head_dim), int(n_state),
                                 int(groups), _ptr(seq_first), _ptr(seq_slots), _ptr(state), state.stride(0),
                                 int(state_offset), _ptr(out), int(xbc.shape[0] > 4 * seq_slots.numel()), _stream()),
           ("ssd_scan(heads={}, P={}, N={})", n_heads, head_dim, n_state))
    return out


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, parts: int, eps: float,
                     out: torch.Tensor, gate_after: bool = False) -> torch.Tensor:
    """out = unit_rms_per_part(y * silu(z)) * weight, or with ``gate_after`` unit_rms_per_part(y) * weight * silu(z):
    ``y`` float32, ``z`` and ``out`` in the compute dtype."""
    _need_cuda(y, z, weight, out)
    inner = y.shape[1]
    if (y.dtype != torch.float32 or y.stride(1) != 1 or z.stride(1) != 1 or out.stride(1) != 1 or z.dtype != out.dtype
            or z.shape != y.shape or out.shape != y.shape or weight.dtype != torch.float32 or weight.numel() != inner
            or inner % parts):
        raise KernelError("gated_group_norm: inputs do not fit")
    _check(library().mu_gated_group_norm(_ptr(y), y.stride(0), _ptr(z), z.stride(0), _ptr(weight), y.shape[0], inner,
                                         int(parts), float(eps), _ptr(out), out.stride(0), _is_bf16(out), _stream(),
                                         int(gate_after)),
           "gated_group_norm")
    return out


# ------------------------------------------------------------------ whole-projection norms, the stream's join
def qkv_norm_rows(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], q_weight: torch.Tensor,
                  k_weight: Optional[torch.Tensor], eps: float, n_kv_heads: int, vdim: int, value_norm: bool, tok_pos,
                  tok_seq, block_table: Optional[torch.Tensor], page_tokens: int, rows: Optional[torch.Tensor],
                  first: Optional[torch.Tensor] = None, first_mode: int = 0, mix: float = 0.0) -> None:
    """Queries [T, q_width] to unit rms over the whole row times ``q_weight``, in place; keys [T, k_width] likewise
    with ``k_weight`` into the token's cache row, each kv head's values (to unit rms over ``vdim`` with
    ``value_norm``) behind them.  ``first`` (float32 [T, kv heads * vdim]): ``first_mode`` 1 stores the values
    there, 2 blends them as (1 - mix) v + mix first before the cache.  ``k`` and ``v`` None: queries only."""
    _need_cuda(q, k, v, q_weight, k_weight, tok_pos, tok_seq, block_table, rows, first)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        _i32(t, name)
    if q.dim() != 2 or q.stride(1) != 1 or q_weight.dtype != torch.float32 or q_weight.numel() != q.shape[1]:
        raise KernelError("qkv_norm_rows: queries are [T, q_width] with unit inner stride and a float32 weight of q_width")
    k_width = 0
    if k is not None:
        k_width = k.shape[1]
        if (k.dtype != q.dtype or v.dtype != q.dtype or rows.dtype != q.dtype or k.stride(1) != 1 or v.stride(1) != 1
                or v.shape[1] != n_kv_heads * vdim or not rows.is_contiguous() or rows.shape[1] != page_tokens
                or rows.shape[2] != k_width + n_kv_heads * vdim or k_weight.dtype != torch.float32
                or k_weight.numel() != k_width):
            raise KernelError("qkv_norm_rows: keys, values, weight and cache rows do not fit the sizes given")
    if first_mode and (first is None or first.dtype != torch.float32 or not first.is_contiguous()
                       or tuple(first.shape) != (q.shape[0], n_kv_heads * vdim)):
        raise KernelError("qkv_norm_rows: the shared values are contiguous float32 [T, kv heads * vdim]")
    _check(library().mu_qkv_norm_rows(_ptr(q), q.stride(0), _ptr(k), k.stride(0) if k is not None else 0, _ptr(v),
                                      v.stride(0) if v is not None else 0, _ptr(q_weight), _ptr(k_weight), float(eps),
                                      q.shape[0], q.shape[1], int(k_width), int(n_kv_heads), int(vdim), int(value_norm),
                                      _ptr(first), int(first_mode), float(mix), _ptr(tok_pos), _ptr(tok_seq),
                                      _ptr(block_table), block_table.shape[1] if block_table is not None else 0,
                                      int(page_tokens), _ptr(rows), _is_bf16(q), _stream()),
           ("qkv_norm_rows(q={}, k={})", q.shape[1], k_width))


def residual_add_norm(x: torch.Tensor, y: Optional[torch.Tensor], mult: float, weight: Optional[torch.Tensor],
                      eps: float, out: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """x += mult * y on the float32 stream (``y`` None: nothing is added), then out = x / rms(x) * weight in
    ``out``'s dtype (``weight`` None: the addition only)."""
    _need_cuda(x, y, weight, out)
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("residual_add_norm: the stream is float32 [rows, n] with unit inner stride")
    if y is not None and (y.dtype != torch.float32 or y.shape != x.shape or y.stride(1) != 1):
        raise KernelError("residual_add_norm: the sublayer's output is float32 and shaped like the stream")
    if weight is not None and (weight.dtype != torch.float32 or weight.numel() != x.shape[1] or not weight.is_contiguous()
                               or out is None or out.shape != x.shape or out.stride(1) != 1):
        raise KernelError("residual_add_norm: a float32 weight of n values and an output shaped like the stream")
    _check(library().mu_residual_add_norm(_ptr(x), x.stride(0), _ptr(y), y.stride(0) if y is not None else 0, float(mult),
                                          _ptr(weight), float(eps), x.shape[0], x.shape[1], _ptr(out),
                                          out.stride(0) if out is not None else 0,
                                          _is_bf16(out) if out is not None else 0, _stream()),
           ("residual_add_norm(n={})", x.shape[1]))
    return out


def xielu(a: torch.Tensor, pair: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The activation with a quadratic branch above zero and an exponential one below, slopes from ``pair`` (two
    float32 on the device, each through softplus); ``out`` may be ``a``."""
    out = a if out is None else out
    _need_cuda(a, pair, out)
    if (a.dim() != 2 or a.shape != out.shape or a.dtype != out.dtype or a.stride(1) != 1 or out.stride(1) != 1
            or pair.dtype != torch.float32 or pair.numel() != 2 or not pair.is_contiguous()):
        raise KernelError("xielu takes [rows, n] views of one dtype with unit inner stride and two float32 numbers")
    _check(library().mu_xielu(_ptr(a), a.stride(0), _ptr(pair), _ptr(out), out.stride(0), a.shape[0], a.shape[1],
                              _is_bf16(a), _stream()), "xielu")
    return out


# ------------------------------------------------------------------ gated delta rule
def delta_scan_max_dk() -> int:
    return int(library().mu_delta_scan_max_dk())


def delta_prepare(qkv: torch.Tensor, b_raw: torch.Tensor, a_raw: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                  n_heads: int, n_kv_heads: int, dk: int, q_scale: float, kq: torch.Tensor, beta: torch.Tensor,
                  decay: torch.Tensor) -> None:
    """Finishes the convolved rows ``qkv`` (float32 [T, 2 * kv heads * dk + ...]) in place: q and k of every kv head to
    unit vectors (eps 1e-6 under the root), q times ``q_scale``; ``kq`` [T, kv heads] their product; per head
    ``beta`` = sigmoid(b_raw) and ``decay`` = exp(-exp(A_log) softplus(a_raw + dt_bias)), float32 [T, heads]."""
    _need_cuda(qkv, b_raw, a_raw, a_log, dt_bias, kq, beta, decay)
    T = qkv.shape[0]
    if (qkv.dtype != torch.float32 or not qkv.is_contiguous() or b_raw.dtype != a_raw.dtype or b_raw.stride(1) != 1
            or a_raw.stride(1) != 1 or tuple(b_raw.shape) != (T, n_heads) or tuple(a_raw.shape) != (T, n_heads)):
        raise KernelError("delta_prepare: rows or raw gates do not fit")
    for t, n in ((a_log, n_heads), (dt_bias, n_heads), (kq, T * n_kv_heads), (beta, T * n_heads), (decay, T * n_heads)):
        if t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous():
            raise KernelError("delta_prepare: float32 per-head parameters and outputs of the sizes given")
    _check(library().mu_delta_prepare(_ptr(qkv), qkv.shape[1], _ptr(b_raw), b_raw.stride(0), _ptr(a_raw), a_raw.stride(0),
                                      _ptr(a_log), _ptr(dt_bias), T, int(n_heads), int(n_kv_heads), int(dk),
                                      float(q_scale), _ptr(kq), _ptr(beta), _ptr(decay), _is_bf16(b_raw), _stream()),
           "delta_prepare")


def delta_scan(qkv: torch.Tensor, kq: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, n_heads: int,
               n_kv_heads: int, dk: int, dv: int, seq_first, seq_slots, state: torch.Tensor, state_offset: int,
               out: torch.Tensor) -> torch.Tensor:
    """The recurrence S = decay S; u = beta (v - S^T k); S += k u^T; o = S^T q per (sequence, head) over the step's
    tokens, from and to ``state[slot][state_offset:]`` (heads x dv x dk float32); ``out`` float32 [T, heads * dv]."""
    _need_cuda(qkv, kq, beta, decay, seq_first, seq_slots, state, out)
    _i32(seq_first, "seq_first"); _i32(seq_slots, "seq_slots")
    T = qkv.shape[0]
    if (qkv.dtype != torch.float32 or not qkv.is_contiguous() or qkv.shape[1] != 2 * n_kv_heads * dk + n_heads * dv
            or out.dtype != torch.float32 or not out.is_contiguous() or tuple(out.shape) != (T, n_heads * dv)
            or state.dtype != torch.float32 or state.stride(1) != 1
            or state.shape[1] < state_offset + n_heads * dv * dk):
        raise KernelError("delta_scan: rows, state or output do not fit")
    _check(library().mu_delta_scan(_ptr(qkv), qkv.shape[1], _ptr(kq), _ptr(beta), _ptr(decay), seq_slots.numel(),
                                   int(n_heads), int(n_kv_heads), int(dk), int(dv), _ptr(seq_first), _ptr(seq_slots),
                                   _ptr(state), state.stride(0), int(state_offset), _ptr(out),
                                   int(T > 4 * seq_slots.numel()), _stream()),
           ("delta_scan(heads={}, dk={}, dv={})", n_heads, dk, dv))
    return out


def sigmoid_gate(o: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """o *= sigmoid(g) in place ([rows, width] views of one dtype with unit inner stride), in float32."""
    _need_cuda(o, g)
    if o.shape != g.shape or o.dtype != g.dtype or o.dim() != 2 or o.stride(1) != 1 or g.stride(1) != 1:
        raise KernelError("sigmoid_gate takes two [rows, width] views of one dtype with unit inner stride")
    _check(library().mu_sigmoid_gate(_ptr(o), o.stride(0), _ptr(g), g.stride(0), o.shape[0], o.shape[1], _is_bf16(o),
                                     _stream()), "sigmoid_gate")
    return o


def rotary(x: torch.Tensor, out: torch.Tensor, tok_pos: torch.Tensor, freqs: torch.Tensor, magnitude: float,
           n_heads: int, dims: int, width: int, x_head_stride: int, out_head_stride: int) -> torch.Tensor:
    """Rotates, for every token (row) and head, ``dims`` entries of the head's slice of ``width`` entries: entry i
    with entry i + dims/2 by the angle position * freqs[i], cos and sin times ``magnitude``; entries past ``dims``
    are copied.  ``x`` and ``out`` are views whose first element is head 0's first entry; they may be the same."""
    _need_cuda(x, out, tok_pos, freqs)
    _i32(tok_pos, "tok_pos")
    if freqs.dtype != torch.float32 or freqs.numel() < dims // 2 or dims % 2:
        raise KernelError("rotary wants dims / 2 float32 frequencies")
    _check(library().mu_rotary(_ptr(x), x.stride(0), int(x_head_stride), _is_bf16(x), _ptr(out), out.stride(0),
                               int(out_head_stride), _is_bf16(out), _ptr(tok_pos), _ptr(freqs), float(magnitude),
                               x.shape[0], int(n_heads), int(dims), int(width), _stream()), ("rotary(dims={})", dims))
    return out


def latent_append(dkv: Optional[torch.Tensor], norm_weight: Optional[torch.Tensor], eps: float, freqs: torch.Tensor,
                  magnitude: float, rot_dims: int, kv_rank: int, rot_dim: int, tok_pos, tok_seq,
                  block_table: torch.Tensor, page_tokens: int, rows: torch.Tensor, queries=None,
                  pairs: bool = False) -> None:
    """Per token: the RMS norm of the first ``kv_rank`` values of ``dkv`` and the rotation of the last ``rot_dim``
    go to the token's row of the latent cache ``rows`` [pages, page_tokens, kv_rank + rot_dim].

    ``queries`` = (q, q_head_stride, qa, qa_head_stride, n_heads): the same launch rotates every head's ``rot_dim``
    entries (views whose first element is head 0's first rotated entry) from ``q`` into the float32 ``qa``.  With
    ``dkv`` None only that is done (a layer that reads another layer's cache).  ``pairs``: entry 2i turns with
    entry 2i + 1 instead of entry i with entry i + rot_dims / 2."""
    _need_cuda(dkv, norm_weight, freqs, tok_pos, tok_seq, block_table, rows)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        _i32(t, name)
    if dkv is not None:
        if dkv.dtype != rows.dtype or dkv.stride(1) != 1 or dkv.shape[1] != kv_rank + rot_dim or not rows.is_contiguous():
            raise KernelError("latent_append: the projection and the cache must share a dtype and the row width")
        if rows.shape[1] != page_tokens or rows.shape[2] != kv_rank + rot_dim:
            raise KernelError("latent_append: the cache is not [pages, page_tokens, kv_rank + rot_dim]")
    q = qa = None
    qs = qas = heads = 0
    if queries is not None:
        q, qs, qa, qas, heads = queries
        _need_cuda(q, qa)
        if q.dtype != rows.dtype or qa.dtype != torch.float32 or q.stride(1) != 1 or qa.stride(1) != 1:
            raise KernelError("latent_append: queries in the cache's dtype, rotated queries as float32")
    elif dkv is None:
        raise KernelError("latent_append: nothing to do")
    n_tokens = dkv.shape[0] if dkv is not None else q.shape[0]
    _check(library().mu_latent_append(_ptr(dkv), dkv.stride(0) if dkv is not None else 0, _ptr(norm_weight), float(eps),
                                      _ptr(freqs), float(magnitude), int(rot_dims), int(kv_rank), int(rot_dim),
                                      _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), block_table.shape[1],
                                      int(page_tokens), n_tokens, _ptr(rows), _is_bf16(rows), _ptr(q),
                                      q.stride(0) if q is not None else 0, int(qs), _ptr(qa),
                                      qa.stride(0) if qa is not None else 0, int(qas), int(heads), _stream(),
                                      int(pairs)),
           "latent_append")


def latent_attention(q: torch.Tensor, rows: torch.Tensor, block_table: torch.Tensor, page_tokens: int, tok_pos, tok_seq,
                     n_heads: int, kv_rank: int, scale: float, out: torch.Tensor, n_splits: int = 1,
                     part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                     tiles: Optional[torch.Tensor] = None, single_tokens: bool = False,
                     tensor_cores: Optional[bool] = None, sink: Optional[torch.Tensor] = None,
                     two_term_weights: bool = False) -> torch.Tensor:
    """Attention of float32 queries [T, n_heads, width] over the latent rows 0..position of each token's sequence;
    ``out`` [T, n_heads * kv_rank] receives the weighted sums of the rows' first ``kv_rank`` values.

    bfloat16 caches at the sizes ``mu_latent_attention_mma`` takes go to the tensor cores when the step says how its
    tokens group: ``tiles`` (int32 [n, 2]: first flat token and count <= 64 of runs of tokens of one sequence) or
    ``single_tokens`` (every token is the one token of its sequence); ``tensor_cores`` false keeps the CUDA-core
    kernel.  ``n_splits`` > 1 (single-token steps) cuts each sequence's rows into parts that are merged afterwards.
    ``sink`` (float32, one per head): exp(sink[h]) is added to head h's softmax denominator, with no value behind it.
    ``two_term_weights``: on the tensor cores the softmax's weights enter the second product as two bfloat16 terms
    (the rounded weight and what the rounding left), so that they act with some 16 bits instead of 8."""
    _need_cuda(q, rows, block_table, tok_pos, tok_seq, out, part_o, part_ml, tiles, sink)
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != n_heads or not sink.is_contiguous()):
        raise KernelError("latent_attention: the sink is one contiguous float32 per head")
    _i32(tiles, "tiles")
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        _i32(t, name)
    width = rows.shape[2]
    n_tokens = q.shape[0]
    if q.dtype != torch.float32 or not q.is_contiguous() or q.numel() != n_tokens * n_heads * width:
        raise KernelError("latent_attention queries must be contiguous float32 [T, heads, width]")
    if out.dtype != rows.dtype or out.stride(1) != 1 or out.shape[1] != n_heads * kv_rank or not rows.is_contiguous():
        raise KernelError("latent_attention output must be [T, heads * kv_rank] in the cache's dtype")
    if n_splits > 1:
        need = n_tokens * n_heads * n_splits
        if (part_o is None or part_ml is None or part_o.numel() < need * kv_rank or part_ml.numel() < need * 2
                or part_o.dtype != torch.float32 or part_ml.dtype != torch.float32):
            raise KernelError("split attention needs float32 scratch for its partial results")
    if tensor_cores is None:
        tensor_cores = LATENT_TC
    if (tensor_cores and rows.dtype == torch.bfloat16 and (tiles is not None or single_tokens)
            and out.stride(0) % 2 == 0 and library().mu_latent_attention_mma_fits(int(kv_rank), int(width), int(page_tokens))):
        if tiles is not None:
            n_splits = 1
        what = ("latent_attention_mma(heads={}, kv_rank={}, width={})", n_heads, kv_rank, width)
        _check(library().mu_latent_attention_mma(
            _ptr(q), _ptr(rows), _ptr(block_table), block_table.shape[1], _ptr(tok_pos), _ptr(tok_seq), _ptr(tiles),
            tiles.shape[0] if tiles is not None else 0, n_tokens, int(n_heads), int(kv_rank), int(width), float(scale),
            int(n_splits), _ptr(out), out.stride(0), _ptr(part_o), _ptr(part_ml), _stream(), _ptr(sink),
            int(two_term_weights)), what)
        if n_splits > 1:
            _check(library().mu_latent_merge(_ptr(part_o), _ptr(part_ml), n_tokens, int(n_heads), int(kv_rank),
                                             int(n_splits), _ptr(out), out.stride(0), 1, _stream(), _ptr(sink)), what)
        return out
    _check(library().mu_latent_attention(_ptr(q), _ptr(rows), _ptr(block_table), block_table.shape[1], int(page_tokens),
                                         _ptr(tok_pos), _ptr(tok_seq), n_tokens, int(n_heads), int(kv_rank), int(width),
                                         float(scale), int(n_splits), _ptr(out), out.stride(0), _ptr(part_o),
                                         _ptr(part_ml), _is_bf16(rows), _stream(), _ptr(sink)),
           ("latent_attention(heads={}, kv_rank={}, width={})", n_heads, kv_rank, width),
           launches=2 if n_splits > 1 else 1)
    return out


# ------------------------------------------------------------------ routed experts
def moe_tile_rows() -> int:
    return int(library().mu_moe_tile_rows())


def moe_route(h: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], top: int, scale: float,
              expert_of: torch.Tensor, weight_of: torch.Tensor, softmax: bool = False, renormalize: bool = False,
              renorm_eps: float = 0.0, gate_weight: Optional[torch.Tensor] = None,
              gate_out: Optional[torch.Tensor] = None) -> None:
    """Router of a feed-forward of experts: logits in float32 from the rows of ``h``, sigmoid (or softmax) scores,
    the ``top`` experts by score + correction into ``expert_of`` [T, top] int32, score * scale into ``weight_of``
    (with ``renormalize`` divided by the chosen scores' sum + ``renorm_eps``).  ``gate_weight`` (float32 [hidden])
    with ``gate_out`` (float32 [T]): the same launch leaves sigmoid(gate_weight . h) per token, a shared expert's gate."""
    _need_cuda(h, router, correction, expert_of, weight_of, gate_weight, gate_out)
    if (gate_weight is None) != (gate_out is None):
        raise KernelError("moe_route: a shared expert's gate needs its weight and a place for the result")
    if gate_weight is not None and (gate_weight.dtype != torch.float32 or not gate_weight.is_contiguous()
                                    or gate_weight.numel() != h.shape[1] or gate_out.dtype != torch.float32
                                    or gate_out.numel() < h.shape[0] or not gate_out.is_contiguous()):
        raise KernelError("moe_route: the gate weight is float32 [hidden], its result float32 [T]")
    n_experts, hidden = router.shape
    if router.dtype != torch.float32 or not router.is_contiguous() or h.shape[1] != hidden or h.stride(1) != 1:
        raise KernelError("moe_route takes rows [T, hidden] and a contiguous float32 router [experts, hidden]")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != n_experts):
        raise KernelError("moe_route: the correction is one float32 per expert")
    _i32(expert_of, "expert_of")
    _check(library().mu_moe_route(_ptr(h), h.stride(0), _is_bf16(h), _ptr(router), _ptr(correction), h.shape[0], hidden,
                                  n_experts, int(top), float(scale), int(softmax), int(renormalize), _ptr(expert_of),
                                  _ptr(weight_of), _stream(), float(renorm_eps), _ptr(gate_weight), _ptr(gate_out)),
           ("moe_route(experts={}, top={})", n_experts, top))


def moe_tc_ok(x_dtype: torch.dtype, k1: int, k2: int) -> bool:
    """Whether the experts' products of a bfloat16 layer go to the tensor cores (both inner sizes multiples of 8)."""
    return LATENT_TC and x_dtype == torch.bfloat16 and k1 % 8 == 0 and k2 % 8 == 0


def moe_group(expert_of: torch.Tensor, n_experts: int, slot_of: torch.Tensor, pair_of: torch.Tensor,
              tile_info: torch.Tensor, n_tiles: torch.Tensor, tile_rows: int = 0, n_real: int = 0) -> None:
    """Groups the (token, expert) pairs by expert: a slot per pair, and the list of tiles of up to ``tile_rows``
    slots per expert (0: the CUDA-core product's tile).  ``n_real`` > 0: the experts from ``n_real`` on have no
    matrices (identity experts); their pairs get slot -1 and no tile."""
    _need_cuda(expert_of, slot_of, pair_of, tile_info, n_tiles)
    for t, name in ((expert_of, "expert_of"), (slot_of, "slot_of"), (pair_of, "pair_of"), (tile_info, "tile_info"),
                    (n_tiles, "n_tiles")):
        _i32(t, name)
    _check(library().mu_moe_group(_ptr(expert_of), expert_of.numel(), int(n_experts), _ptr(slot_of), _ptr(pair_of),
                                  _ptr(tile_info), _ptr(n_tiles), int(tile_rows) or moe_tile_rows(), _stream(),
                                  int(n_real)),
           "moe_group")


def moe_gemm(x: torch.Tensor, pair_of: Optional[torch.Tensor], top: int, w1: torch.Tensor, w2: Optional[torch.Tensor],
             tile_info: torch.Tensor, n_tiles: torch.Tensor, max_tiles: int, out: torch.Tensor,
             tensor_cores: Optional[bool] = None, tile_rows: int = 0, act: Optional[str] = None) -> torch.Tensor:
    """out[slot] = act(W1[e] x[row]) (or silu(W1[e] x[row]) * W2[e] x[row] with ``w2``) for every slot of every expert e
    (``act``: None or ``relu2``);
    ``w1``/``w2`` [experts, n, k]; rows of ``x`` by the slot's token (``pair_of``) or by slot.  bfloat16 operands
    with 16-byte aligned rows go to the tensor cores unless ``tensor_cores`` is false.  ``tile_rows``: what
    ``moe_group`` was given (the CUDA-core product takes its own tile only)."""
    _need_cuda(x, pair_of, w1, w2, tile_info, n_tiles, out)
    if w1.dim() != 3 or not w1.is_contiguous() or w1.dtype != x.dtype or x.stride(1) != 1 or x.shape[1] != w1.shape[2]:
        raise KernelError("moe_gemm takes rows [*, k] and contiguous weights [experts, n, k] of one dtype")
    if w2 is not None and (w2.shape != w1.shape or w2.dtype != w1.dtype or not w2.is_contiguous()):
        raise KernelError("moe_gemm: the two weight stacks must agree")
    if out.stride(1) != 1 or out.shape[1] != w1.shape[1]:
        raise KernelError("moe_gemm output has the wrong shape or stride")
    if tensor_cores is None:
        tensor_cores = LATENT_TC
    if act not in (None, "none", "relu2") or (act == "relu2" and w2 is not None):
        raise KernelError(f"moe_gemm: activation '{act}' is not taken (relu2 without a second weight stack, or none)")
    code = ACT_CODES[act]
    tile_rows = int(tile_rows) or moe_tile_rows()
    if (tensor_cores and x.dtype == torch.bfloat16 and w1.shape[2] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w1.data_ptr() % 16 == 0 and (w2 is None or w2.data_ptr() % 16 == 0)):
        _check(library().mu_moe_gemm_mma(_ptr(x), x.stride(0), _ptr(pair_of), int(top), _ptr(w1), _ptr(w2),
                                         w1.stride(0), w1.stride(1), _ptr(tile_info), _ptr(n_tiles), int(max_tiles),
                                         tile_rows, w1.shape[1], w1.shape[2], _ptr(out), out.stride(0), _is_bf16(out),
                                         _stream(), code), ("moe_gemm_mma(n={}, k={})", w1.shape[1], w1.shape[2]))
        return out
    if tile_rows != moe_tile_rows():
        raise KernelError(f"the CUDA-core experts' product takes tiles of {moe_tile_rows()} slots, got {tile_rows}")
    _check(library().mu_moe_gemm(_ptr(x), x.stride(0), _ptr(pair_of), int(top), _ptr(w1), _ptr(w2),
                                 w1.stride(0), w1.stride(1), _ptr(tile_info), _ptr(n_tiles), int(max_tiles),
                                 w1.shape[1], w1.shape[2], _ptr(out), out.stride(0), _is_bf16(x), _is_bf16(out),
                                 _stream(), code), ("moe_gemm(n={}, k={})", w1.shape[1], w1.shape[2]))
    return out


def heads_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_head_stride: int, out_head_stride: int,
               gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, h, :] = W[h] x[t, h, :] for every row t and head h: ``w`` [heads, n, k]; ``x`` / ``out`` views whose first
    element is head 0's first entry, a head's slice ``x_head_stride`` / ``out_head_stride`` elements after the head
    before.  bfloat16 operands with aligned slices run as ONE launch on the tensor cores; anything else head by head
    through ``linear``.  ``gate`` (laid out as ``out``): out *= sigmoid(gate), in the product's epilogue where that
    launch runs, as a launch of its own otherwise."""
    _need_cuda(x, w, out, gate)
    heads, n, k = w.shape
    if (LATENT_TC and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and k % 8 == 0
            and x.stride(0) % 8 == 0 and x_head_stride % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.stride(1) == 1 and out.stride(1) == 1):
        fused = gate is not None and gate.dtype == torch.bfloat16 and gate.stride(1) == 1 and gate.shape == out.shape
        _check(library().mu_heads_gemm(_ptr(x), x.stride(0), int(x_head_stride), _ptr(w), w.stride(0), w.stride(1),
                                       x.shape[0], heads, n, k, _ptr(out), out.stride(0), int(out_head_stride),
                                       _is_bf16(out), _ptr(gate) if fused else None, gate.stride(0) if fused else 0,
                                       _stream()), ("heads_gemm(heads={}, n={}, k={})", heads, n, k))
        if gate is not None and not fused:
            sigmoid_gate(out, gate)
        return out
    for h in range(heads):
        linear(x[:, h * x_head_stride: h * x_head_stride + k], w[h], out=out[:, h * out_head_stride: h * out_head_stride + n])
    if gate is not None:
        sigmoid_gate(out, gate)
    return out


def moe_combine(y: torch.Tensor, slot_of: torch.Tensor, weight_of: torch.Tensor, top: int, out: torch.Tensor,
                identity_rows: Optional[torch.Tensor] = None, shared: Optional[torch.Tensor] = None,
                shared_gate: Optional[torch.Tensor] = None, add: bool = False) -> torch.Tensor:
    """out[t] (+)= sum over the token's choices, in their order, of weight * y[slot]; float32.  A choice without a
    slot (an identity expert, slot -1) contributes weight * ``identity_rows[t]`` (the experts' input rows, compute
    dtype).  ``shared`` (float32 [T, width]) is added to every token, times ``shared_gate[t]`` if given.  ``add``:
    the result is added to what ``out`` holds."""
    _need_cuda(y, slot_of, weight_of, out, identity_rows, shared, shared_gate)
    if y.dtype != torch.float32 or out.dtype != torch.float32 or y.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("moe_combine works on float32 rows with unit inner stride")
    if identity_rows is not None and (identity_rows.shape != out.shape or identity_rows.stride(1) != 1):
        raise KernelError("moe_combine: the identity rows are shaped like the output, unit inner stride")
    if shared is not None and (shared.dtype != torch.float32 or shared.shape != out.shape or shared.stride(1) != 1):
        raise KernelError("moe_combine: the shared expert's rows are float32 and shaped like the output")
    if shared_gate is not None and (shared is None or shared_gate.dtype != torch.float32 or not shared_gate.is_contiguous()
                                    or shared_gate.numel() < out.shape[0]):
        raise KernelError("moe_combine: the shared expert's gate is float32 [T] and needs the shared rows")
    _check(library().mu_moe_combine(_ptr(y), y.stride(0), _ptr(slot_of), _ptr(weight_of), out.shape[0], int(top),
                                    out.shape[1], _ptr(out), out.stride(0), _stream(), _ptr(identity_rows),
                                    identity_rows.stride(0) if identity_rows is not None else 0,
                                    _is_bf16(identity_rows) if identity_rows is not None else 0, _ptr(shared),
                                    shared.stride(0) if shared is not None else 0, _ptr(shared_gate), int(add)),
           "moe_combine")
    return out


def rms_norm_pair(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, eps: float, out1: torch.Tensor,
                  out2: torch.Tensor) -> None:
    """out1 = x / sqrt(mean(x^2) + eps) * w1 and out2 = the same rows * w2: two norms of one float32 stream in one
    pass (one statistic).  Both outputs float32 or both bfloat16."""
    _need_cuda(x, w1, w2, out1, out2)
    n = x.shape[1]
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("rms_norm_pair input must be float32 [rows, n] with unit inner stride")
    for w in (w1, w2):
        if w.dtype != torch.float32 or not w.is_contiguous() or w.numel() != n:
            raise KernelError("rms_norm_pair takes contiguous float32 weights of n values")
    if out1.dtype != out2.dtype or out1.shape != x.shape or out2.shape != x.shape or out1.stride(1) != 1 or out2.stride(1) != 1:
        raise KernelError("rms_norm_pair outputs are of one dtype and shaped like the input")
    _check(library().mu_rms_norm_pair(_ptr(x), x.stride(0), _ptr(w1), _ptr(w2), float(eps), _ptr(out1), out1.stride(0),
                                      _ptr(out2), out2.stride(0), _is_bf16(out1), x.shape[0], n, _stream()),
           ("rms_norm_pair(n={})", n))


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) on float32 rows, in place."""
    _need_cuda(x)
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1 or not cap > 0.0:
        raise KernelError("softcap takes float32 [rows, n] with unit inner stride and a positive cap")
    _check(library().mu_softcap(_ptr(x), x.stride(0), x.shape[0], x.shape[1], float(cap), _stream()), "softcap")
    return x


def moe_combine_tanh(y: torch.Tensor, slot_of: torch.Tensor, weight_of: torch.Tensor, top: int, weight: torch.Tensor,
                     bias: Optional[torch.Tensor], alpha: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] += tanh(alpha v) * weight + bias with v = the token's weighted sum of its experts' rows (``moe_combine``
    and ``dynamic_tanh(add=True)`` in one launch)."""
    _need_cuda(y, slot_of, weight_of, weight, bias, alpha, out)
    if y.dtype != torch.float32 or out.dtype != torch.float32 or y.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("moe_combine_tanh works on float32 rows with unit inner stride")
    _check(library().mu_moe_combine_tanh(_ptr(y), y.stride(0), _ptr(slot_of), _ptr(weight_of), out.shape[0], int(top),
                                         out.shape[1], _ptr(weight), _ptr(bias), _ptr(alpha), _ptr(out), out.stride(0),
                                         _stream()), "moe_combine_tanh")
    return out


# ------------------------------------------------------------------------ GEMM
def _gemm_args(a, w, bias, residual, out, out_dtype):
    _need_cuda(a, w, bias, residual, out)
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        raise KernelError(f"gemm shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}")
    if a.dtype != w.dtype:
        raise KernelError(f"gemm operands differ in dtype: {a.dtype} and {w.dtype}")
    if a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm operands must have unit stride along k")
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if out.shape != (m, n) or out.stride(1) != 1:
        raise KernelError("gemm output has the wrong shape or stride")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != n):
        raise KernelError("gemm bias must be float32 of length n")
    if residual is not None and (residual.dtype != torch.float32 or residual.shape != (m, n)
                                 or residual.stride(1) != 1):
        raise KernelError("gemm residual must be float32 [m, n]")
    return m, n, k, out


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
              act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """out = act(a @ w^T + bias) + residual on CUDA cores, any shape, any of the
    two dtypes; with float32 operands this is the true 32-bit product."""
    m, n, k, out = _gemm_args(a, w, bias, residual, out, out_dtype or a.dtype)
    _check(library().mu_gemm_simt(
        _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), m, n, k, a.stride(0), w.stride(0),
        out.stride(0), residual.stride(0) if residual is not None else 0, ACT_CODES[act],
        _is_bf16(a), _is_bf16(out), _stream()), ("gemm_simt({}x{}x{})", m, n, k))
    return out


_status = {}


def status_word(device) -> torch.Tensor:
    """A device word that kernels with bounded waits write to when a wait runs
    out (it stays 0 otherwise); ``check_status`` reads it."""
    word = _status.get(device)
    if word is None:
        word = _status[device] = _status[str(device)] = torch.zeros(1, dtype=torch.int32, device=device)
        _split_workspace(device)
    return word


def _rows_kernel(m: int, n: int, k: int) -> bool:
    """Whether a product of m rows goes to ``mu_gemm_rows``: 33 to 64 rows always; 17 to 32 rows where the
    weights are 16 million or more (the output head, which that kernel streams faster than the few-rows
    kernel does at that many rows).  Up to 16 rows the few-rows kernel with the norm folded in stays ahead
    inside a step, where its weights are on their way while the kernels before it end."""
    return 33 <= m <= 64 or (17 <= m <= 32 and n * k >= (1 << 24))


def _split_workspace(device) -> None:
    """Room for tensor-core products that are cut along k (few output tiles,
    long k: a batch of 33 to 128 single tokens): partial tiles for one tile per
    SM at the widest tile, and a ticket per tile.  Set once per device, at the
    first use of a kernel with a status word, hence never inside a capture."""
    parts = scratch("gemm_tc_parts", device, sm_count(device) * 128 * 256, torch.float32)
    tickets = zeroed_workspace("gemm_tc_tickets", device, 4 * 1024)
    _check(library().mu_gemm_tc_split_workspace(parts.data_ptr(), parts.numel() * 4, tickets.data_ptr(),
                                                tickets.numel() // 4), "gemm_tc_split_workspace", launches=0)


_WAITS = {1: "tensor-core product: loads", 2: "tensor-core product: tensor cores",
          3: "tensor-core product: epilogue", 4: "single-token attention: a page copy",
          5: "prompt attention: loads", 6: "prompt attention: tensor cores", 7: "prompt attention: softmax",
          8: "streamed product: a weight copy"}


def raise_status(device, code: int) -> None:
    """Clears the status word and raises for the wait that ran out."""
    word = _status.get(str(torch.device(device)))
    if word is not None:
        word.zero_()
    raise KernelError(f"a kernel gave up a bounded wait ({_WAITS.get(code, f'code {code}')}); the results of "
                      "the steps since the last check are not valid")


def check_status(device="cuda:0") -> None:
    """Raises if a kernel gave up a bounded wait since the last check (this
    synchronises with the device)."""
    word = _status.get(str(torch.device(device)))
    if word is not None:
        code = int(word.item())
        if code != 0:
            raise_status(device, code)


def tc_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether gemm_tc takes this product (alignment rules of its TMA loads)."""
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
            act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
            tile: int = 0, splits: int = -1) -> torch.Tensor:
    """The product on the tcgen05 tensor cores (TMA loads, accumulator in tensor memory).
    ``tile``: width of the output tiles (64, 128, 256; 0: the library chooses); ``splits``: parts that k
    is cut into (-1: the library chooses; 0 or 1: none)."""
    m, n, k, out = _gemm_args(a, w, bias, residual, out, out_dtype or a.dtype)
    _check(library().mu_gemm_tc(
        _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), m, n, k, a.stride(0), w.stride(0),
        out.stride(0), residual.stride(0) if residual is not None else 0, ACT_CODES[act],
        _is_bf16(out), int(tile), int(splits), _ptr(status_word(a.device)), _stream()),
        ("gemm_tc({}x{}x{})", m, n, k))
    return out


def gemm_rows(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
              act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
              splits: int = 0) -> torch.Tensor:
    """The product for up to 64 rows on the tcgen05 tensor cores: tiles of 16 output columns, a block per
    tile, k cut over a thread-block cluster where the tiles are few (``splits`` blocks per tile, 0: chosen
    by the library), the parts added in rank order in the first block's shared memory."""
    m, n, k, out = _gemm_args(a, w, bias, residual, out, out_dtype or a.dtype)
    _check(library().mu_gemm_rows(
        _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), m, n, k, a.stride(0), w.stride(0),
        out.stride(0), residual.stride(0) if residual is not None else 0, ACT_CODES[act],
        _is_bf16(out), int(splits), _ptr(status_word(a.device)), _stream()), ("gemm_rows({}x{}x{})", m, n, k))
    return out


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """The product for a few rows (single-token steps): streams the weights once
    through mma.sync with the weight rows as the wide operand."""
    m, n, k, out = _gemm_args(a, w, bias, residual, out, out_dtype or a.dtype)
    _check(library().mu_gemm_skinny(
        _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), m, n, k, a.stride(0), w.stride(0),
        out.stride(0), residual.stride(0) if residual is not None else 0, ACT_CODES[act],
        _is_bf16(out), _stream()), ("gemm_skinny({}x{}x{})", m, n, k))
    return out


# ------------------------------------------------------------------- attention
def kv_append(k: torch.Tensor, v: torch.Tensor, tok_pos, tok_seq, block_table: torch.Tensor,
              page_tokens: int, n_kv_heads: int, head_dim: int, kv_pages: torch.Tensor,
              tiles: Optional[torch.Tensor] = None) -> None:
    """Copies keys and values of this step's tokens ([T, n_kv_heads * head_dim]
    views, unit inner stride) into their pages (values transposed: dimension-major
    within a page).  ``tiles`` (int32 [n, 2]: first flat token and count <= 64 of
    runs of tokens of one sequence) lets prompt values be written a tile at a time."""
    _need_cuda(k, v, tok_pos, tok_seq, block_table, kv_pages)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        _i32(t, name)
    if k.dtype != kv_pages.dtype or v.dtype != kv_pages.dtype:
        raise KernelError("keys, values and the cache must share a dtype")
    if k.stride(1) != 1 or v.stride(1) != 1:
        raise KernelError("keys and values must have unit inner stride")
    _check(library().mu_kv_append(
        _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(tok_pos), _ptr(tok_seq),
        _ptr(block_table), block_table.shape[1], page_tokens, k.shape[0], n_kv_heads, head_dim,
        _ptr(kv_pages), _is_bf16(kv_pages), _ptr(tiles), tiles.shape[0] if tiles is not None else 0, _stream()),
        ("kv_append(head_dim={})", head_dim))


def attention(q: torch.Tensor, out: torch.Tensor, kv_pages: torch.Tensor, block_table: torch.Tensor,
              page_tokens: int, tok_pos, tok_seq, n_heads: int, n_kv_heads: int, head_dim: int,
              scale: float, window: int = 0, n_splits: int = 1, split_keys: int = 0,
              part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of each query token ([T, n_heads * head_dim] view) over the
    cached keys first..its position; writes ``out`` [T, n_heads * head_dim]."""
    _need_cuda(q, out, kv_pages, block_table, tok_pos, tok_seq, part_o, part_ml)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        _i32(t, name)
    if q.dtype != kv_pages.dtype or out.dtype != kv_pages.dtype:
        raise KernelError("queries, output and the cache must share a dtype")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("queries and output must have unit inner stride")
    n_tokens = q.shape[0]
    if n_splits > 1:
        need_o, need_ml = n_tokens * n_heads * n_splits * head_dim, n_tokens * n_heads * n_splits * 2
        if (part_o is None or part_ml is None or part_o.numel() < need_o or part_ml.numel() < need_ml
                or part_o.dtype != torch.float32 or part_ml.dtype != torch.float32):
            raise KernelError("split attention needs float32 scratch for its partial results")
    _check(library().mu_attention(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kv_pages), _ptr(block_table),
        block_table.shape[1], page_tokens, _ptr(tok_pos), _ptr(tok_seq), n_tokens,
        n_heads, n_kv_heads, head_dim, float(scale), int(window), int(n_splits), int(split_keys),
        _ptr(part_o), _ptr(part_ml), _is_bf16(kv_pages), _stream()),
        ("attention(heads={}/{}, head_dim={})", n_heads, n_kv_heads, head_dim), launches=2 if n_splits > 1 else 1)
    return out


# -------------------------------------------------------------------- sampling
def _status_args(status_to: Optional[torch.Tensor], device):
    if status_to is None:
        return None, None
    _i32(status_to, "status_to")
    if not status_to.is_cuda or status_to.numel() != 1:
        raise KernelError("status_to must be one int32 word on the device")
    return _ptr(status_word(device)), _ptr(status_to)


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, feed=None,
           status_to: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First maximum of each row.  ``feed`` = (token_ids, tok_pos, last_pos): the
    tokens also become the next single-token step's inputs and the positions
    (if not None) move on by one (what ``advance`` does, without its launch).
    ``status_to``: a device word that receives the kernels' status word, so
    that one copy brings tokens and status to the host."""
    _need_cuda(logits, out)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 [rows, vocab] with unit inner stride")
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    ws = zeroed_workspace("argmax", logits.device, 2 * n * 8)
    ids, pos, last = feed if feed is not None else (None, None, 0)
    _check(library().mu_argmax(_ptr(logits), logits.stride(0), n, vocab, _ptr(out), _ptr(ws), _ptr(ids), _ptr(pos),
                               int(last), *_status_args(status_to, logits.device), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, seed: int,
           request_ids: Optional[torch.Tensor], draw_index: torch.Tensor,
           out: Optional[torch.Tensor] = None, feed=None, status_to: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row by temperature / top-k; ``draw_index`` (int32 per row)
    counts the draws of each request and is advanced by one.  ``feed`` and
    ``status_to`` as for ``argmax``."""
    _need_cuda(logits, request_ids, draw_index, out)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 [rows, vocab] with unit inner stride")
    if request_ids is not None and request_ids.dtype != torch.int64:
        raise KernelError("request_ids must be int64")
    _i32(draw_index, "draw_index")
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(library().mu_sample(_ptr(logits), logits.stride(0), n, vocab, float(temperature), int(top_k),
                               int(seed) & ((1 << 64) - 1), _ptr(request_ids), _ptr(draw_index), _ptr(out),
                               _ptr(feed[0]) if feed else None, _ptr(feed[1]) if feed else None,
                               int(feed[2]) if feed else 0, *_status_args(status_to, logits.device), _stream()),
           "sample")
    return out


class NormedInput:
    """The LayerNorm of (rows of) a float32 matrix that has not been computed
    yet: a product kernel that can make it on the fly takes this instead of a
    tensor; anything else calls ``materialize``."""

    def __init__(self, x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float,
                 out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None):
        self.x, self.gamma, self.beta, self.eps, self.out_dtype, self.rows = x, gamma, beta, eps, out_dtype, rows
        self._value = None

    @property
    def n_rows(self) -> int:
        return self.rows.numel() if self.rows is not None else self.x.shape[0]

    def materialize(self) -> torch.Tensor:
        if self._value is None:
            self._value = layernorm(self.x, self.gamma, self.beta, self.eps, self.out_dtype, rows=self.rows)
        return self._value

    def materialize_copy(self) -> torch.Tensor:
        """The norm computed for an onlooker; what a product does with this input stays as it was."""
        return layernorm(self.x, self.gamma, self.beta, self.eps, self.out_dtype, rows=self.rows)


def gemm_skinny_ln(x: NormedInput, w: torch.Tensor, bias, act, residual, out, out_dtype) -> torch.Tensor:
    """act(LayerNorm(x) @ w^T + bias) + residual with the norm made inside the product kernel."""
    _need_cuda(x.x, w, bias, residual, out, x.rows)
    m, k, n = x.n_rows, x.x.shape[1], w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or w.dtype, device=w.device)
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != n):
        raise KernelError("gemm bias must be float32 of length n")
    if residual is not None and (residual.dtype != torch.float32 or residual.shape != (m, n)):
        raise KernelError("gemm residual must be float32 [m, n]")
    _check(library().mu_gemm_skinny_ln(
        _ptr(x.x), x.x.stride(0), _ptr(x.rows), _ptr(x.gamma), _ptr(x.beta), float(x.eps), _ptr(w), _ptr(bias),
        _ptr(residual), _ptr(out), m, n, k, w.stride(0), out.stride(0),
        residual.stride(0) if residual is not None else 0, ACT_CODES[act], _is_bf16(out), _stream()),
        ("gemm_skinny_ln({}x{}x{})", m, n, k))
    return out


def _stream_kernel(m: int, n: int, k: int, ldw: int, with_norm: bool, device) -> bool:
    """Whether a product of up to 16 rows goes to ``mu_gemm_stream``: very many output columns (an output head:
    what the few-rows kernel would run as blocks of 128 columns each), weight rows one after another, and a k
    short enough for two tiles of 64 weight rows to share an SM's shared memory."""
    return (m <= 16 and n >= 256 * sm_count(device)
            and bool(library().mu_gemm_stream_fits(int(m), int(k), int(ldw), 1 if with_norm else 0)))


def gemm_stream(x, w: torch.Tensor, bias=None, act=None, out=None, out_dtype=None) -> torch.Tensor:
    """act(x @ w^T + bias) for up to 16 rows and very many output columns, the weights streamed through shared
    memory by bulk copies.  ``x``: bfloat16 [m, k], or a ``NormedInput`` (the norm is made inside the kernel)."""
    normed = isinstance(x, NormedInput)
    if normed:
        _need_cuda(x.x, w, bias, out, x.rows)
        m, k = x.n_rows, x.x.shape[1]
    else:
        _need_cuda(x, w, bias, out)
        m, k = x.shape
    n = w.shape[0]
    if w.dtype != torch.bfloat16 or w.shape[1] != k or w.stride(1) != 1:
        raise KernelError("gemm_stream needs bfloat16 weights [n, k] with unit stride along k")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or w.dtype, device=w.device)
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != n):
        raise KernelError("gemm bias must be float32 of length n")
    _check(library().mu_gemm_stream(
        None if normed else _ptr(x), 0 if normed else x.stride(0),
        _ptr(x.x) if normed else None, x.x.stride(0) if normed else 0, _ptr(x.rows) if normed else None,
        _ptr(x.gamma) if normed else None, _ptr(x.beta) if normed else None, float(x.eps) if normed else 0.0,
        _ptr(w), _ptr(bias), _ptr(out), m, n, k, w.stride(0), out.stride(0), ACT_CODES[act], _is_bf16(out),
        _ptr(status_word(w.device)), _stream()), ("gemm_stream({}x{}x{})", m, n, k))
    return out


SKINNY_LN_SMEM = 160 * 1024          # the limit of mu_gemm_skinny_ln (gemm_skinny.cuh)

_sm_counts = {}


def sm_count(device) -> int:
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def decode_ok(head_dim: int) -> bool:
    """Whether the one-launch single-token attention kernels take this head size
    (multiples of 16 up to 256: their key rows are read in 16-byte pieces); other
    sizes append first and then run the general kernel."""
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def decode_tc_ok(q, k_new, v_new, kv_pages, page_tokens: int, n_heads: int, n_kv_heads: int,
                 head_dim: int) -> bool:
    """Whether the tensor-core single-token attention takes this case (else the
    CUDA-core kernel does): bfloat16, head sizes 32, 64, 96 and 128, at most 16 query
    heads per kv head, 16-byte aligned rows.  MU_B200_ATT_TC=0 switches it off."""
    if not ATT_TC:
        return False
    if kv_pages.dtype != torch.bfloat16 or page_tokens != 64 or head_dim not in (32, 64, 96, 128):
        return False
    if n_heads % n_kv_heads != 0 or n_heads // n_kv_heads > 16:
        return False
    for t in (q, k_new, v_new):
        if t is not None and (t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0):
            return False
    return True


def decode_block_shape(blocks: int, sms: int) -> int:
    """The shape of the tensor-core single-token attention kernel's blocks for this many (sequence, kv head)
    pairs, as the code ``mu_attention_decode_tc`` takes.  No more blocks than SMs: large ones (6), all pages of
    a sequence in flight at once; up to twice as many: three groups of two warps, two blocks an SM (3); more:
    small ones, three an SM (2; the large ones would run in waves).  Very few: four (24) or two (12) large
    blocks share a sequence's pages as a cluster, while the clusters fill two thirds or half of the SMs at
    most (a cluster is placed within one part of the chip, so a fuller grid of clusters runs in waves)."""
    if 6 * blocks <= sms:
        return 24
    if 4 * blocks <= sms:
        return 12
    if blocks <= sms:
        return 6
    return 3 if blocks <= 2 * sms else 2


def attention_decode(q: torch.Tensor, k_new: Optional[torch.Tensor], v_new: Optional[torch.Tensor],
                     out: torch.Tensor, kv_pages: torch.Tensor, block_table: torch.Tensor, page_tokens: int,
                     tok_pos, tok_seq, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                     window: int, n_splits: int, warps: int = 0) -> torch.Tensor:
    """Single-token attention, one launch: appends ``k_new`` / ``v_new`` (if
    given), attends page by page, merges in shared memory.  ``n_splits``: how
    many warps share a sequence's pages (its page count is a good choice; at most
    16 are used).  ``tok_seq`` None: token t is sequence t.  ``warps``: the shape of a
    block (tensor-core kernel: 2, 3 or 6 groups of warps, 12 or 24 for six groups in
    each of two or four blocks that share a sequence; CUDA-core kernel: an upper bound
    on its warps); 0: chosen here."""
    _need_cuda(q, k_new, v_new, out, kv_pages, block_table, tok_pos, tok_seq)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        _i32(t, name)
    n_tokens = q.shape[0]
    if decode_tc_ok(q, k_new, v_new, kv_pages, page_tokens, n_heads, n_kv_heads, head_dim):
        if not warps:
            warps = decode_block_shape(n_tokens * n_kv_heads, sm_count(q.device))
        _check(library().mu_attention_decode_tc(
            _ptr(q), q.stride(0), _ptr(k_new), k_new.stride(0) if k_new is not None else 0, _ptr(v_new),
            v_new.stride(0) if v_new is not None else 0, _ptr(out), out.stride(0), _ptr(kv_pages),
            _ptr(block_table), block_table.shape[1], page_tokens, _ptr(tok_pos), _ptr(tok_seq), n_tokens,
            n_heads, n_kv_heads, head_dim, float(scale), int(window), int(warps),
            _ptr(status_word(q.device)), _stream()),
            ("attention_decode_tc(heads={}/{}, head_dim={})", n_heads, n_kv_heads, head_dim))
        return out
    _check(library().mu_attention_decode(
        _ptr(q), q.stride(0), _ptr(k_new), k_new.stride(0) if k_new is not None else 0, _ptr(v_new),
        v_new.stride(0) if v_new is not None else 0, _ptr(out), out.stride(0), _ptr(kv_pages),
        _ptr(block_table), block_table.shape[1], page_tokens, _ptr(tok_pos), _ptr(tok_seq), n_tokens,
        n_heads, n_kv_heads, head_dim, float(scale), int(window), int(n_splits), int(warps), _is_bf16(kv_pages),
        _stream()),
        ("attention_decode(heads={}/{}, head_dim={})", n_heads, n_kv_heads, head_dim))
    return out


def prefill_ok(q: torch.Tensor, head_dim: int, page_tokens: int) -> bool:
    """Whether the tensor-core prompt attention takes this case."""
    return (q.dtype == torch.bfloat16 and page_tokens == 64 and head_dim % 16 == 0 and 16 <= head_dim <= 128
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


def attention_prefill(q: torch.Tensor, out: torch.Tensor, kv_pages: torch.Tensor, block_table: torch.Tensor,
                      page_tokens: int, tok_pos, tok_seq, tiles: torch.Tensor, n_heads: int, n_kv_heads: int,
                      head_dim: int, scale: float, window: int = 0) -> torch.Tensor:
    """Flash-style causal attention of prompt tokens on tensor cores.  ``tiles``
    int32 [n, 2]: first flat query index and query count (<= 64) of each tile;
    the kernel's blocks take them in this order, so the tiles with the most keys
    should come first."""
    _need_cuda(q, out, kv_pages, block_table, tok_pos, tok_seq, tiles)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table"), (tiles, "tiles")):
        _i32(t, name)
    counter = zeroed_workspace("attention_prefill_items", q.device, 8)
    _check(library().mu_attention_prefill(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kv_pages), _ptr(block_table), block_table.shape[1],
        page_tokens, _ptr(tok_pos), _ptr(tok_seq), _ptr(tiles), tiles.shape[0], n_heads, n_kv_heads, head_dim,
        float(scale), int(window), _ptr(counter), _stream()), ("attention_prefill(heads={}/{}, head_dim={})", n_heads, n_kv_heads, head_dim))
    return out


def prefill_tc_ok(q: torch.Tensor, out: torch.Tensor, head_dim: int, page_tokens: int) -> bool:
    """Whether the tcgen05 prompt attention takes this case: bfloat16, head size
    64, pages of 64, query and output rows 16-byte aligned.  MU_B200_PREFILL_TC=0
    switches it off (the mma.sync kernel then runs)."""
    if not PREFILL_TC:
        return False
    return (q.dtype == torch.bfloat16 and head_dim == 64 and page_tokens == 64 and q.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0)


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, kv_pages: torch.Tensor, block_table: torch.Tensor,
                         page_tokens: int, tok_pos, tok_seq, tiles: torch.Tensor, n_heads: int, n_kv_heads: int,
                         head_dim: int, scale: float, window: int = 0, k_new: Optional[torch.Tensor] = None,
                         v_new: Optional[torch.Tensor] = None, append_tiles: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of prompt tokens on the tcgen05 tensor cores (TMA loads,
    scores and outputs in tensor memory).  ``tiles`` int32 [n, 2]: first flat
    query index and query count (<= 128) of each tile, longest tiles first.
    With ``k_new`` / ``v_new`` the step's keys and values are appended to the
    cache first, in the same call (``append_tiles``: tiles of <= 64 tokens)."""
    _need_cuda(q, out, kv_pages, block_table, tok_pos, tok_seq, tiles, k_new, v_new, append_tiles)
    for t, name in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (block_table, "block_table"), (tiles, "tiles"),
                    (append_tiles, "append_tiles")):
        _i32(t, name)
    if k_new is not None and (k_new.dtype != kv_pages.dtype or v_new is None or v_new.dtype != kv_pages.dtype
                              or k_new.stride(1) != 1 or v_new.stride(1) != 1):
        raise KernelError("keys, values and the cache must share a dtype; unit stride within a row")
    _check(library().mu_attention_prefill_tc(
        _ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), _ptr(kv_pages), kv_pages.shape[0],
        _ptr(block_table), block_table.shape[1], page_tokens, _ptr(tok_pos), _ptr(tok_seq), _ptr(tiles),
        tiles.shape[0], n_heads, n_kv_heads, head_dim, float(scale), int(window),
        _ptr(k_new), k_new.stride(0) if k_new is not None else 0, _ptr(v_new),
        v_new.stride(0) if v_new is not None else 0, _ptr(append_tiles),
        append_tiles.shape[0] if append_tiles is not None else 0,
        _ptr(status_word(q.device)), _stream()),
        ("attention_prefill_tc(heads={}/{}, head_dim={})", n_heads, n_kv_heads, head_dim),
        launches=2 if k_new is not None else 1)
    return out


_scratch = {}


def scratch(name: str, device, numel: int, dtype) -> torch.Tensor:
    """A device buffer kept per purpose, device and dtype that only ever grows
    (a buffer it outgrows is kept alive: a recorded graph may still point at it)."""
    key = (name, device, dtype)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < numel:
        if buf is not None:
            _retired.append(buf)
        buf = _scratch[key] = torch.empty(max(numel, 1), dtype=dtype, device=device)
    return buf


def _layernorm_gemm_tc(x: "NormedInput", weight, bias, act, residual, out, out_dtype):
    """The norm and the tensor-core product of it from one call into the library
    (two launches), for more than 64 rows of bfloat16; None if the case is not its."""
    m, k = x.n_rows, x.x.shape[1]
    n = weight.shape[0]
    if (m <= 64 or x._value is not None or weight.dtype != torch.bfloat16 or x.out_dtype != torch.bfloat16
            or x.x.dtype != torch.float32 or not x.x.is_contiguous() or weight.dim() != 2 or weight.shape[1] != k
            or weight.stride(1) != 1 or k % 8 != 0 or weight.stride(0) % 8 != 0 or weight.data_ptr() % 16 != 0):
        return None
    if not (x.x.is_cuda and weight.is_cuda and x.gamma.dtype == torch.float32
            and (x.beta is None or x.beta.dtype == torch.float32)):
        return None
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or torch.bfloat16, device=weight.device)
    elif out.shape != (m, n) or out.stride(1) != 1 or not out.is_cuda:
        raise KernelError("gemm output has the wrong shape, stride or device")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != n or not bias.is_cuda):
        raise KernelError("gemm bias must be float32 of length n on the device")
    ldr = 0
    if residual is not None:
        if residual.dtype != torch.float32 or residual.shape != (m, n) or residual.stride(1) != 1 or not residual.is_cuda:
            raise KernelError("gemm residual must be float32 [m, n] on the device")
        ldr = residual.stride(0)
    _i32(x.rows, "rows")
    normed = scratch("layernorm_out", weight.device, m * k, torch.bfloat16)
    _check(library().mu_layernorm_gemm_tc(
        x.x.data_ptr(), _ptr(x.rows), x.gamma.data_ptr(), _ptr(x.beta), float(x.eps), normed.data_ptr(),
        weight.data_ptr(), _ptr(bias), _ptr(residual), out.data_ptr(), m, n, k, weight.stride(0), out.stride(0),
        ldr, ACT_CODES[act], _is_bf16(out), status_word(weight.device).data_ptr(), _stream()),
        ("layernorm_gemm_tc({}x{}x{})", m, n, k), launches=2)
    return out


# ------------------------------------------------------ a whole layer of a prompt step in one call
class PromptLayerArgs(ctypes.Structure):
    """Everything ``mu_prompt_layer`` needs; the layout is ``MuPromptLayerArgs`` of prompt_layer.cu."""
    _fields_ = (
        [(n, _c_p) for n in ("x", "normed", "qkv", "attn", "inner_buf", "tok_pos", "tok_seq", "block_table",
                             "tiles_wide", "tiles", "status", "stream", "kv_pages", "ln1_gamma", "ln1_beta",
                             "qkv_weight", "qkv_bias", "out_weight", "out_bias", "ln2_gamma", "ln2_beta",
                             "up_weight", "up_bias", "down_weight", "down_bias")]
        + [(n, _c_ll) for n in ("n_cache_pages", "ld_qkv_weight", "ld_out_weight", "ld_up_weight", "ld_down_weight")]
        + [(n, _c_f) for n in ("eps1", "eps2", "scale")]
        + [(n, _c_int) for n in ("n_tokens", "hidden", "inner", "n_heads", "n_kv_heads", "head_dim", "window", "act",
                                 "max_pages", "page_tokens", "n_tiles_wide", "n_tiles", "owns_cache")])


_PROMPT_LAUNCHES = ("", "the norm and the q | k | v product", "the cache append and the attention", "the output projection",
                    "the norm and the feed-forward's first product", "the feed-forward's second product")


def prompt_layer(args: PromptLayerArgs) -> None:
    """Issues the launches of one pre-norm layer of a prompt step (eight kernels) from one call."""
    lib = library()
    fn = lib.mu_prompt_layer
    if fn.argtypes is None:
        if lib.mu_prompt_layer_args_size() != ctypes.sizeof(PromptLayerArgs):
            raise KernelError("the layer-call layout of the Python side and of the kernel library differ")
        fn.argtypes, fn.restype = [ctypes.POINTER(PromptLayerArgs)], _c_int
    args.stream = _stream()
    code = fn(ctypes.byref(args))
    if code != 0:
        raise KernelError(f"prompt layer, {_PROMPT_LAUNCHES[min(code // 100, 5)]}: "
                          f"{_ERRORS.get(code % 100, f'error {code % 100}')}")
    global launch_count
    launch_count += 7 + int(bool(args.owns_cache))


# -------------------------------------------------------------------- dispatch
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(x @ weight^T + bias) + residual through the kernel that fits the
    dtype and the shape.  float32 operands always take the CUDA-core kernel.
    ``x`` may be a ``NormedInput``: with few rows and bfloat16 weights the norm is
    made inside the product kernel, otherwise it is computed first."""
    if isinstance(x, NormedInput) and weight.dtype == torch.bfloat16 and _rows_kernel(x.n_rows, *weight.shape):
        x = x.materialize()          # a very wide product: the norm as a launch of its own costs less than it saves
    if isinstance(x, NormedInput):
        k_in = x.x.shape[1]
        # the few-rows kernel keeps the normed rows (8, 16 or 32 of them), gamma and beta in shared memory
        fits = 8 * (1 if x.n_rows <= 8 else 2 if x.n_rows <= 16 else 4) * (k_in + 8) * 2 + 8 * k_in <= SKINNY_LN_SMEM
        if (weight.dtype == torch.bfloat16 and x.out_dtype == torch.bfloat16 and x.n_rows <= 32 and fits
                and k_in % 8 == 0 and weight.stride(0) % 8 == 0 and weight.data_ptr() % 16 == 0
                and x.x.dtype == torch.float32 and x.x.stride(1) == 1):
            if (residual is None and x.x.stride(0) % 4 == 0 and x.x.data_ptr() % 16 == 0
                    and _stream_kernel(x.n_rows, weight.shape[0], k_in, weight.stride(0), True, weight.device)):
                return gemm_stream(x, weight, bias, act, out, out_dtype)      # an output head
            return gemm_skinny_ln(x, weight, bias, act, residual, out, out_dtype)
        fused = _layernorm_gemm_tc(x, weight, bias, act, residual, out, out_dtype)
        if fused is not None:
            return fused
        x = x.materialize()
    # One pass over what the kernels need, then straight to the library (this is the call a prompt
    # step makes a hundred times): the shapes must agree here; alignment, strides and sizes that a
    # kernel cannot take come back from the library as an error code.
    if x.dim() != 2 or weight.dim() != 2:
        raise KernelError(f"gemm shapes do not agree: a {tuple(x.shape)}, w {tuple(weight.shape)}")
    m, k = x.shape
    n, kw = weight.shape
    dtype = x.dtype
    if k != kw or dtype != weight.dtype or x.stride(1) != 1 or weight.stride(1) != 1:
        raise KernelError(f"gemm operands do not agree: a {tuple(x.shape)} {dtype}, w {tuple(weight.shape)} "
                          f"{weight.dtype}, unit stride along k needed")
    if not (x.is_cuda and weight.is_cuda):
        raise KernelError("math_utils_b200 kernels run on CUDA tensors only")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or dtype, device=x.device)
    elif out.shape != (m, n) or out.stride(1) != 1 or not out.is_cuda:
        raise KernelError("gemm output has the wrong shape, stride or device")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != n or not bias.is_cuda):
        raise KernelError("gemm bias must be float32 of length n on the device")
    ldr = 0
    if residual is not None:
        if residual.dtype != torch.float32 or residual.shape != (m, n) or residual.stride(1) != 1 or not residual.is_cuda:
            raise KernelError("gemm residual must be float32 [m, n] on the device")
        ldr = residual.stride(0)
    lda, ldw = x.stride(0), weight.stride(0)
    pa, pw = x.data_ptr(), weight.data_ptr()
    pb = None if bias is None else bias.data_ptr()
    pr = None if residual is None else residual.data_ptr()
    lib = library()
    code = ACT_CODES[act]
    tensor_cores = (dtype == torch.bfloat16 and k % 8 == 0 and lda % 8 == 0 and ldw % 8 == 0
                    and pa % 16 == 0 and pw % 16 == 0)
    # 33 to 64 rows, and fewer where the weights are very many (the output head): the tcgen05 kernel for few
    # rows (weights as the wide operand, k cut over a cluster); up to 32 rows otherwise the mma.sync kernel
    # that streams weights straight into fragments; more than 64 rows the large tcgen05 kernel
    if tensor_cores and _rows_kernel(m, n, k):
        _check(lib.mu_gemm_rows(pa, pw, pb, pr, out.data_ptr(), m, n, k, lda, ldw, out.stride(0), ldr, code,
                                _is_bf16(out), 0, status_word(x.device).data_ptr(), _stream()),
               ("gemm_rows({}x{}x{})", m, n, k))
    elif tensor_cores and m <= 32:
        _check(lib.mu_gemm_skinny(pa, pw, pb, pr, out.data_ptr(), m, n, k, lda, ldw, out.stride(0), ldr, code,
                                  _is_bf16(out), _stream()), ("gemm_skinny({}x{}x{})", m, n, k))
    elif tensor_cores:
        _check(lib.mu_gemm_tc(pa, pw, pb, pr, out.data_ptr(), m, n, k, lda, ldw, out.stride(0), ldr, code,
                              _is_bf16(out), 0, -1, status_word(x.device).data_ptr(), _stream()),
               ("gemm_tc({}x{}x{})", m, n, k))
    else:
        _check(lib.mu_gemm_simt(pa, pw, pb, pr, out.data_ptr(), m, n, k, lda, ldw, out.stride(0), ldr, code,
                                _is_bf16(x), _is_bf16(out), _stream()), ("gemm_simt({}x{}x{})", m, n, k))
    return out
