"""Functional CUDA twins of the reference's codec primitives, on torch tensors.

Each function takes CUDA tensors, validates like the reference's numpy function of
the same name (``ValueError`` on bad shapes), and calls the C ABI with raw device
pointers on the current stream.  PyTorch is only the owner of device memory here.
"""

from __future__ import annotations

import torch

from . import _lib
from ._lib import DT_BF16, DT_F16, DT_F32

_DTYPES = {torch.float16: DT_F16, torch.bfloat16: DT_BF16, torch.float32: DT_F32}


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _need_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: the EXL3 path has no CPU implementation")


def as_u16(t: torch.Tensor) -> torch.Tensor:
    """int16 / uint16 storage of packed trellis words (bit pattern is what matters)."""
    if t.dtype in (torch.int16, torch.uint16):
        return t
    raise ValueError(f"packed trellis must be (u)int16, got {t.dtype}")


class Workspace:
    """Per-device scratch for the matmul entry points: the status word, the arrival counters and
    partial sums of split column blocks, and the rotated activations.  One per device, grown on
    demand; calls that share it are ordered by the stream they run on.

    A buffer that has been handed out is never freed: CUDA graphs captured earlier and work on
    other streams keep its raw address, so when a later call needs more room a new buffer is
    allocated and the old ones stay alive (and are still looked at by `status`).  Growth does
    not migrate captured graphs — they keep using the buffer they were captured with."""

    _per_device: dict[int, "Workspace"] = {}
    _retired: dict[int, list["Workspace"]] = {}

    def __init__(self, device: torch.device, nbytes: int):
        lib = _lib.load()
        self.device = device
        self.nbytes = int(nbytes)
        self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        _lib.check(lib.exl3_workspace_init(self.buf.data_ptr(), self.nbytes, _stream(device)),
                   "exl3_workspace_init")

    @classmethod
    def get_bytes(cls, device: torch.device, nbytes: int) -> "Workspace":
        """The device's workspace; a larger one replaces it when it is too small (the old buffer
        stays allocated, see the class docstring)."""
        idx = device.index if device.index is not None else torch.cuda.current_device()
        ws = cls._per_device.get(idx)
        if ws is None or ws.nbytes < nbytes:
            if ws is not None:
                cls._retired.setdefault(idx, []).append(ws)
            floor = int(_lib.load().exl3_workspace_bytes(16, 32768))
            ws = Workspace(torch.device("cuda", idx), max(int(nbytes), floor, ws.nbytes if ws else 0))
            cls._per_device[idx] = ws
        return ws

    _need: dict[tuple[int, int], int] = {}

    @classmethod
    def get(cls, device: torch.device, rows: int, in_features: int) -> "Workspace":
        # the size question goes to the library once per (rows, in) and the answer is kept: this
        # sits on the per-call host path of every decode GEMV
        key = (rows, in_features)
        need = cls._need.get(key)
        if need is None:
            need = cls._need[key] = int(_lib.load().exl3_workspace_bytes(rows, in_features))
        idx = device.index
        ws = cls._per_device.get(idx) if idx is not None else None
        if ws is not None and ws.nbytes >= need:
            return ws
        return cls.get_bytes(device, need)

    def _status_one(self) -> int:
        import ctypes
        out = ctypes.c_int(0)
        _lib.check(_lib.load().exl3_workspace_status(self.buf.data_ptr(), ctypes.byref(out),
                                                     _stream(self.device)), "exl3_workspace_status")
        return out.value

    def status(self) -> int:
        """OR of the sticky status words of this device's workspace and of every buffer it has
        replaced (0 = no bounded wait of any kernel ever gave up)."""
        idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
        st = self._status_one()
        for old in self._retired.get(idx, []):
            if old is not self:
                st |= old._status_one()
        return st


def unpack_trellis(packed: torch.Tensor, k: int) -> torch.Tensor:
    """(tiles_k, tiles_n, 16K) packed words -> (tiles_k, tiles_n, 256) int16 codewords
    (ponyexl3/ref/trellis.py:205-214)."""
    _need_cuda(packed, "packed")
    if packed.ndim != 3:
        raise ValueError(f"expected 3D packed trellis, got {tuple(packed.shape)}")
    if not 1 <= k <= 8:
        raise ValueError(f"K must be in [1, 8], got {k}")
    if packed.shape[-1] != 16 * k:
        raise ValueError(f"expected last dim {16 * k}, got {packed.shape[-1]}")
    packed = as_u16(packed).contiguous()
    out = torch.empty(packed.shape[:2] + (256,), dtype=torch.int16, device=packed.device)
    n = packed.shape[0] * packed.shape[1]
    if n == 0:
        return out
    _lib.check(_lib.load().exl3_unpack(packed.data_ptr(), n, k, out.data_ptr(),
                                       _stream(packed.device)), "exl3_unpack")
    return out


def quantize_tiles(w: torch.Tensor, k: int, cb: int = 0, max_pins: int = 4,
                   max_tiles_in_flight: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Exact trellis search of 16x16 tiles (quantize_tile_reference,
    ponyexl3/convert/reference_search.py:60-87): w (n, 256) float32 in codeword order ->
    (states (n, 256) int16 holding the 16-bit window of every codeword, packed (n, 16K) int16 tiles
    as stored on disk).  Bit-identical to the reference's search.  The converter's side of the
    format: a tile costs 256 steps over 65,536 states, so this is for converting, not for serving."""
    _need_cuda(w, "w")
    if w.ndim != 2 or w.shape[1] != 256:
        raise ValueError(f"expected w of shape (n_tiles, 256), got {tuple(w.shape)}")
    if not 1 <= k <= 8:
        raise ValueError(f"K must be in [1, 8], got {k}")
    w = w.to(torch.float32).contiguous()
    n = w.shape[0]
    states = torch.empty((n, 256), dtype=torch.int16, device=w.device)
    packed = torch.empty((n, 16 * k), dtype=torch.int16, device=w.device)
    if n == 0:
        return states, packed
    lib = _lib.load()
    with torch.cuda.device(w.device):
        in_flight = n if max_tiles_in_flight is None else max(1, min(n, max_tiles_in_flight))
        nbytes = int(lib.exl3_encode_workspace_bytes(in_flight))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
    _lib.check(lib.exl3_encode_tiles(w.data_ptr(), n, k, int(cb), max_pins, states.data_ptr(), packed.data_ptr(),
                                     ws.data_ptr(), nbytes, _stream(w.device)), "exl3_encode_tiles")
    return states, packed


def tile_codeword_order(device=None) -> torch.Tensor:
    """perm (256,) int64: codeword i of a tile sits at tile position perm[i] = row * 16 + col
    (ponyexl3/ref/perm.py:8-26)."""
    i = torch.arange(256, device=device)
    t, j = i >> 3, i & 7
    row = (t & 3) * 2 + (j & 1) + ((j & 2) != 0) * 8
    col = (t >> 2) + ((j & 4) != 0) * 8
    return row * 16 + col


def quantize_inner(inner: torch.Tensor, k: int, cb: int = 0, max_pins: int = 4) -> torch.Tensor:
    """Inner weight matrix (in, out) -> packed trellis (in/16, out/16, 16K) int16: tiles in codeword
    order (ponyexl3/convert/direct.py:409-420), searched by quantize_tiles.  The rotations and
    scales around the inner matrix are the converter's business."""
    _need_cuda(inner, "inner")
    if inner.ndim != 2 or inner.shape[0] % 16 or inner.shape[1] % 16:
        raise ValueError(f"expected a 2-D matrix with dims that are multiples of 16, got {tuple(inner.shape)}")
    ti, to = inner.shape[0] // 16, inner.shape[1] // 16
    tiles = inner.to(torch.float32).reshape(ti, 16, to, 16).permute(0, 2, 1, 3).reshape(ti * to, 256)
    tiles = tiles[:, tile_codeword_order(inner.device)]
    _, packed = quantize_tiles(tiles, k, cb, max_pins)
    return packed.view(ti, to, 16 * k)


def decode_packed_trellis(trellis: torch.Tensor, k: int, cb: int, *, n_offset: int = 0,
                          n_count: int | None = None) -> torch.Tensor:
    """Inner weight matrix (in, n_count) fp16 of a packed trellis, bit-exact with the
    reference (ponyexl3/ref/decode.py:32-81).  For tests and debugging only."""
    _need_cuda(trellis, "trellis")
    if trellis.ndim != 3:
        raise ValueError("trellis must be 3D")
    t_in, t_out, ps = trellis.shape
    if not 1 <= k <= 8:
        raise ValueError(f"K must be in [1, 8], got {k}")
    if ps != 16 * k:
        raise ValueError(f"packed size {ps} != expected {16 * k} for K={k}")
    if n_offset % 128 != 0:
        raise ValueError("n_offset must be divisible by 128")
    n_count = t_out * 16 - n_offset if n_count is None else n_count
    if n_count % 16 or n_offset + n_count > t_out * 16:
        raise ValueError("slice exceeds output features")
    trellis = as_u16(trellis).contiguous()
    w = torch.empty((t_in * 16, n_count), dtype=torch.float16, device=trellis.device)
    if w.numel() == 0:
        return w
    _lib.check(_lib.load().exl3_decode(trellis.data_ptr(), t_in, t_out, k, int(cb), n_offset // 16,
                                       n_count // 16, w.data_ptr(), n_count,
                                       _stream(trellis.device)), "exl3_decode")
    return w


def codebook_table(cb: int, device: torch.device | str = "cuda") -> torch.Tensor:
    """decode_3inst of every 16-bit codeword (ponyexl3/ref/codebook.py:66-91)."""
    device = torch.device(device)
    t = torch.empty(65536, dtype=torch.float16, device=device)
    _lib.check(_lib.load().exl3_codebook_table(int(cb), t.data_ptr(), _stream(device)),
               "exl3_codebook_table")
    return t


def had_r_128(x: torch.Tensor, *, pre_scale: torch.Tensor | None = None,
              post_scale: torch.Tensor | None = None) -> torch.Tensor:
    """fp16( ((x * pre) @ H128/sqrt(128)) * post ) along the last dimension
    (ponyexl3/ref/hadamard.py:50-80); x fp16 / bf16 / fp32, 2-D."""
    _need_cuda(x, "x")
    if x.ndim != 2:
        raise ValueError("had_r_128 expects 2D input (rows, features)")
    if x.shape[1] % 128 != 0:
        raise ValueError(f"feature dim {x.shape[1]} not divisible by 128")
    if x.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {x.dtype}")
    if x.stride(1) != 1:
        x = x.contiguous()
    pre = None if pre_scale is None else pre_scale.to(torch.float16).contiguous()
    post = None if post_scale is None else post_scale.to(torch.float16).contiguous()
    out = torch.empty(x.shape, dtype=torch.float16, device=x.device)
    _lib.check(_lib.load().exl3_hadamard128(
        x.data_ptr(), _DTYPES[x.dtype], x.shape[0], x.shape[1], x.stride(0),
        None if pre is None else pre.data_ptr(), None if post is None else post.data_ptr(),
        out.data_ptr(), _stream(x.device)), "exl3_hadamard128")
    return out


_GLU_FLAGS = {None: 0, "silu": _lib.FLAG_GLU_SILU, "gelu": _lib.FLAG_GLU_GELU}


def gemv(x2d: torch.Tensor, trellis: torch.Tensor, k: int, cb: int, suh: torch.Tensor | None,
         svh: torch.Tensor | None, bias: torch.Tensor | None, *, pdl: bool = False,
         fast_accum: bool = False, out: torch.Tensor | None = None, glu: str | None = None) -> torch.Tensor:
    """The whole linear forward for 1..16 rows in one launch (two for many rows: rotation, then the
    streamed GEMV).  x2d (rows, in) fp16/bf16/fp32 -> (rows, out) fp16.
    glu = "silu" | "gelu": x2d is (rows, 2*in) = [gate | up] and the input is fp16(act(gate) * up)."""
    _need_cuda(x2d, "x")
    rows, in_features = x2d.shape
    if glu is not None:
        in_features //= 2
    t_in, t_out, _ = trellis.shape
    if in_features != t_in * 16 or (glu is not None and x2d.shape[1] != 2 * in_features):
        raise ValueError(f"x has {in_features} features, layer expects {t_in * 16}")
    if x2d.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {x2d.dtype}")
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    ws = Workspace.get(x2d.device, rows, in_features)
    y = out if out is not None else torch.empty((rows, t_out * 16), dtype=torch.float16,
                                                device=x2d.device)
    _lib.check(_lib.load().exl3_gemv(
        x2d.data_ptr(), _DTYPES[x2d.dtype], rows, x2d.stride(0), trellis.data_ptr(), t_in, t_out,
        k, int(cb), None if suh is None else suh.data_ptr(),
        None if svh is None else svh.data_ptr(), None if bias is None else bias.data_ptr(),
        y.data_ptr(), y.stride(0), ws.buf.data_ptr(), ws.nbytes,
        (_lib.FLAG_PDL if pdl else 0) | (_lib.FLAG_FAST_ACCUM if fast_accum else 0) | _GLU_FLAGS[glu],
        _stream(x2d.device)), "exl3_gemv")
    return y


def gemm(x2d: torch.Tensor, trellis: torch.Tensor, k: int, cb: int, suh: torch.Tensor | None,
         svh: torch.Tensor | None, bias: torch.Tensor | None, *,
         out: torch.Tensor | None = None) -> torch.Tensor:
    """The linear forward for any number of rows on the tensor cores (prefill).
    x2d (rows, in) fp16/bf16/fp32 -> (rows, out) fp16."""
    _need_cuda(x2d, "x")
    rows, in_features = x2d.shape
    t_in, t_out, _ = trellis.shape
    if in_features != t_in * 16:
        raise ValueError(f"x has {in_features} features, layer expects {t_in * 16}")
    if x2d.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {x2d.dtype}")
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    lib = _lib.load()
    ws = Workspace.get_bytes(x2d.device, int(lib.exl3_gemm_workspace_bytes(rows, in_features)))
    y = out if out is not None else torch.empty((rows, t_out * 16), dtype=torch.float16,
                                                device=x2d.device)
    _lib.check(lib.exl3_gemm(
        x2d.data_ptr(), _DTYPES[x2d.dtype], rows, x2d.stride(0), trellis.data_ptr(), t_in, t_out,
        k, int(cb), None if suh is None else suh.data_ptr(),
        None if svh is None else svh.data_ptr(), None if bias is None else bias.data_ptr(),
        y.data_ptr(), y.stride(0), ws.buf.data_ptr(), ws.nbytes, 0, _stream(x2d.device)), "exl3_gemm")
    return y


def gemv_blocks(x2d: torch.Tensor, *, xh_rows: int, row_src: torch.Tensor | None,
                suh: torch.Tensor | None, suh_row: torch.Tensor | None, trellis: torch.Tensor, k: int,
                cb: int, blocks: torch.Tensor, rows: int, svh: torch.Tensor | None,
                bias: torch.Tensor | None, y: torch.Tensor, raw_out: bool = False, pdl: bool = False,
                fast_accum: bool = False, glu: str | None = None,
                n_blocks_dev: torch.Tensor | None = None) -> torch.Tensor:
    """Streamed GEMV over a block table (see exl3_gemv_blocks in the header).  `blocks` is an
    int32 CUDA tensor (n_blocks, 4) = phys, xrow, sv_off, y_off; `y` is written in place.
    glu as in gemv: x2d rows are [gate | up].  n_blocks_dev: an int32 CUDA scalar with the number of
    blocks in use (exl3_gemv_blocks_counted); the table's length is then the upper bound."""
    _need_cuda(x2d, "x")
    t_in, t_out_total, _ = trellis.shape
    if x2d.shape[1] != t_in * 16 * (2 if glu is not None else 1):
        raise ValueError(f"x has {x2d.shape[1]} features, layer expects {t_in * 16}")
    if blocks.dtype != torch.int32 or blocks.ndim != 2 or blocks.shape[1] != 4:
        raise ValueError("blocks must be an int32 tensor of shape (n_blocks, 4)")
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    blocks = blocks.contiguous()
    lib = _lib.load()
    ws = Workspace.get(x2d.device, xh_rows, t_in * 16)
    ptr = lambda t: None if t is None else t.data_ptr()
    flags = (_lib.FLAG_PDL if pdl else 0) | (_lib.FLAG_FAST_ACCUM if fast_accum else 0) | _GLU_FLAGS[glu]
    y_stride = y.stride(0) if y.ndim == 2 else 0
    if n_blocks_dev is None:
        _lib.check(lib.exl3_gemv_blocks(
            x2d.data_ptr(), _DTYPES[x2d.dtype], x2d.stride(0), xh_rows, ptr(row_src), ptr(suh),
            ptr(suh_row), trellis.data_ptr(), t_in, t_out_total, k, int(cb), blocks.data_ptr(),
            blocks.shape[0], rows, ptr(svh), ptr(bias), y.data_ptr(), y_stride,
            1 if raw_out else 0, ws.buf.data_ptr(), ws.nbytes, flags, _stream(x2d.device)), "exl3_gemv_blocks")
    else:
        if n_blocks_dev.dtype != torch.int32 or not n_blocks_dev.is_cuda:
            raise ValueError("n_blocks_dev must be an int32 CUDA tensor")
        _lib.check(lib.exl3_gemv_blocks_counted(
            x2d.data_ptr(), _DTYPES[x2d.dtype], x2d.stride(0), xh_rows, ptr(row_src), ptr(suh),
            ptr(suh_row), trellis.data_ptr(), t_in, t_out_total, k, int(cb), blocks.data_ptr(),
            blocks.shape[0], n_blocks_dev.data_ptr(), rows, ptr(svh), ptr(bias), y.data_ptr(), y_stride,
            1 if raw_out else 0, ws.buf.data_ptr(), ws.nbytes, flags, _stream(x2d.device)),
            "exl3_gemv_blocks_counted")
    return y


def gemm_tiles(x2d: torch.Tensor, *, xh_rows: int, row_src: torch.Tensor | None,
               suh: torch.Tensor | None, suh_row: torch.Tensor | None, trellis: torch.Tensor, k: int,
               cb: int, tiles: torch.Tensor, svh: torch.Tensor | None, y: torch.Tensor | None,
               y_row_map: torch.Tensor | None = None, glu: str | None = None,
               xh_rows_dev: torch.Tensor | None = None, peers=None) -> torch.Tensor | None:
    """Tensor-core GEMM over a tile table (see exl3_gemm_tiles in the header).  `tiles` is an
    int32 CUDA tensor (n_tiles, 8); `y` (rows, cols) fp16 is written in place.
    glu: x2d rows are [gate | up] and the input is fp16(act(gate) * up).
    xh_rows_dev: int32 CUDA scalar, rotated rows in use.  peers = (y_ptrs, counter_ptrs, n,
    rows_per_peer, row_stride): the output rows go to the GPUs that own them (y may be None), see
    exl3_gemm_tiles_peers."""
    _need_cuda(x2d, "x")
    t_in, t_out_total, _ = trellis.shape
    if x2d.shape[1] != t_in * 16 * (2 if glu is not None else 1):
        raise ValueError(f"x has {x2d.shape[1]} features, layer expects {t_in * 16}")
    if tiles.dtype != torch.int32 or tiles.ndim != 2 or tiles.shape[1] != 8:
        raise ValueError("tiles must be an int32 tensor of shape (n_tiles, 8)")
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    tiles = tiles.contiguous()
    lib = _lib.load()
    ws = Workspace.get_bytes(x2d.device, int(lib.exl3_gemm_workspace_bytes(xh_rows, t_in * 16)))
    ptr = lambda t: None if t is None else t.data_ptr()
    flags = _GLU_FLAGS[glu]
    if peers is None and xh_rows_dev is None:
        _lib.check(lib.exl3_gemm_tiles(
            x2d.data_ptr(), _DTYPES[x2d.dtype], x2d.stride(0), xh_rows, ptr(row_src), ptr(suh),
            ptr(suh_row), trellis.data_ptr(), t_in, t_out_total, k, int(cb), tiles.data_ptr(),
            tiles.shape[0], ptr(svh), y.data_ptr(), y.stride(0), ptr(y_row_map), ws.buf.data_ptr(), ws.nbytes, flags,
            _stream(x2d.device)), "exl3_gemm_tiles")
        return y
    if peers is None:
        y_ptrs, c_ptrs, n_peers, rows_per_peer, stride = None, None, 0, 0, y.stride(0)
    else:
        y_ptrs, c_ptrs, n_peers, rows_per_peer, stride = peers
    _lib.check(lib.exl3_gemm_tiles_peers(
        x2d.data_ptr(), _DTYPES[x2d.dtype], x2d.stride(0), xh_rows, ptr(xh_rows_dev), ptr(row_src), ptr(suh),
        ptr(suh_row), trellis.data_ptr(), t_in, t_out_total, k, int(cb), tiles.data_ptr(), tiles.shape[0],
        ptr(svh), ptr(y), stride, ptr(y_row_map), y_ptrs, c_ptrs, n_peers, rows_per_peer, ws.buf.data_ptr(),
        ws.nbytes, flags, _stream(x2d.device)), "exl3_gemm_tiles_peers")
    return y


# ---- the caller's side of a decode step (exl3_step.cu) ---------------------------------------

def _flags(pdl: bool) -> int:
    return _lib.FLAG_PDL if pdl else 0


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor | None = None, pdl: bool = False) -> torch.Tensor:
    """In place x <- x + delta (skipped when delta is None); returns fp16 RMSNorm(x) * weight.
    x, delta (rows, n) fp16 with unit column stride."""
    _need_cuda(x, "x")
    rows, n = x.shape
    h = out if out is not None else torch.empty((rows, n), dtype=torch.float16, device=x.device)
    if delta is not None and delta.stride(1) != 1:
        delta = delta.contiguous()
    _lib.check(_lib.load().exl3_add_rmsnorm(
        x.data_ptr(), None if delta is None else delta.data_ptr(), weight.data_ptr(), h.data_ptr(), rows, n,
        x.stride(0), 0 if delta is None else delta.stride(0), h.stride(0), float(eps), _flags(pdl),
        _stream(x.device)),
        "exl3_add_rmsnorm")
    return h


def rope_append(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, k_cache: torch.Tensor,
                v_cache: torch.Tensor, q_heads: int, pos0: int, out: torch.Tensor | None = None,
                pdl: bool = False) -> torch.Tensor:
    """qkv (rows, (q_heads + 2 kv_heads) * 128) -> rotated q (rows, q_heads, 128); rotated k and
    v are written to rows pos0.. of the caches (kv_heads, cache_len, 128)."""
    _need_cuda(qkv, "qkv")
    rows = qkv.shape[0]
    kv_heads, cache_len, hd = k_cache.shape
    if hd != 128 or qkv.shape[1] != (q_heads + 2 * kv_heads) * 128 or qkv.stride(1) != 1:
        raise ValueError("rope_append expects head_dim 128 and a packed q|k|v row")
    q = out if out is not None else torch.empty((rows, q_heads, 128), dtype=torch.float16, device=qkv.device)
    _lib.check(_lib.load().exl3_rope_append(
        qkv.data_ptr(), qkv.stride(0), cos.data_ptr(), sin.data_ptr(), q.data_ptr(), k_cache.data_ptr(),
        v_cache.data_ptr(), rows, q_heads, kv_heads, cache_len, int(pos0), _flags(pdl), _stream(qkv.device)),
        "exl3_rope_append")
    return q


_attn_ws: dict[int, torch.Tensor] = {}


def attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, ctx: int,
                out: torch.Tensor | None = None, pdl: bool = False) -> torch.Tensor:
    """q (rows, q_heads, 128) over caches (kv_heads, cache_len, 128) that already hold the new
    positions ctx .. ctx+rows-1 -> (rows, q_heads * 128); position r sees keys 0 .. ctx + r."""
    _need_cuda(q, "q")
    rows, q_heads, hd = q.shape
    kv_heads, cache_len, _ = k_cache.shape
    lib = _lib.load()
    need = int(lib.exl3_attn_workspace_bytes(rows, q_heads, kv_heads, ctx + rows))
    if need == 0 or hd != 128:
        raise ValueError("unsupported attention shape")
    idx = q.device.index if q.device.index is not None else torch.cuda.current_device()
    ws = _attn_ws.get(idx)
    if ws is None or ws.numel() < need:
        if ws is not None:
            torch.cuda.current_stream(q.device).synchronize()
        ws = torch.empty(need, dtype=torch.uint8, device=q.device)
        _attn_ws[idx] = ws
    y = out if out is not None else torch.empty((rows, q_heads * 128), dtype=torch.float16, device=q.device)
    _lib.check(lib.exl3_attn_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), y.data_ptr(), rows,
                                    q_heads, kv_heads, cache_len, int(ctx), ws.data_ptr(), ws.numel(),
                                    _flags(pdl), _stream(q.device)), "exl3_attn_decode")
    return y


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, pdl: bool = False) -> torch.Tensor:
    """gate_up (rows, 2h) = [gate | up] -> fp16 silu(gate) * up, (rows, h)."""
    _need_cuda(gate_up, "gate_up")
    rows, two_h = gate_up.shape
    h = two_h // 2
    y = out if out is not None else torch.empty((rows, h), dtype=torch.float16, device=gate_up.device)
    _lib.check(_lib.load().exl3_swiglu(gate_up.data_ptr(), gate_up.stride(0), y.data_ptr(), y.stride(0), rows, h,
                                       _flags(pdl), _stream(gate_up.device)), "exl3_swiglu")
    return y


# ---- output exchange over peer memory (exl3_peer.cu) -----------------------------------------

def gemv_peers(x2d: torch.Tensor, trellis: torch.Tensor, k: int, cb: int, suh, svh, bias, *, exchange,
               out_features_total: int, col0: int, pdl: bool = False, defer_wait: bool = False) -> torch.Tensor:
    """exl3_gemv whose output blocks land in every rank's full row (`exchange`: a
    parallel.PeerExchange).  Returns this rank's (rows, out_features_total) row buffer.

    The row is complete once every rank's blocks have arrived.  By default the wait for them is
    launched right behind the GEMV.  With defer_wait=True it is left pending on the exchange: the
    next gemv_peers call folds it into its own kernel (which then must read the pending row, or
    at least run after it is complete), and `exchange.settle()` launches it for any other reader."""
    _need_cuda(x2d, "x")
    rows, in_features = x2d.shape
    t_in, t_out, _ = trellis.shape
    if in_features != t_in * 16:
        raise ValueError(f"x has {in_features} features, layer expects {t_in * 16}")
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    lib = _lib.load()
    ws = Workspace.get(x2d.device, rows, in_features)
    pending = exchange.pending
    _, y_ptrs, c_ptrs, view, my_ctr = exchange.take(rows, out_features_total)
    ptr = lambda t: None if t is None else t.data_ptr()
    flags = _lib.FLAG_PDL if pdl else 0
    rc = _lib.E_UNSUPPORTED
    if pending is not None:
        rc = lib.exl3_gemv_peers_after(
            x2d.data_ptr(), _DTYPES[x2d.dtype], rows, x2d.stride(0), trellis.data_ptr(), t_in, t_out, k, int(cb),
            ptr(suh), ptr(svh), ptr(bias), y_ptrs, c_ptrs, exchange.world, out_features_total, int(col0),
            pending, exchange.world, ws.buf.data_ptr(), ws.nbytes, flags, _stream(x2d.device))
        if rc == 0:
            exchange.pending = None
    if rc == _lib.E_UNSUPPORTED:
        exchange.settle(pdl=pdl)            # the rotation kernel reads x: the row has to be complete first
        rc = lib.exl3_gemv_peers(
            x2d.data_ptr(), _DTYPES[x2d.dtype], rows, x2d.stride(0), trellis.data_ptr(), t_in, t_out, k, int(cb),
            ptr(suh), ptr(svh), ptr(bias), y_ptrs, c_ptrs, exchange.world, out_features_total, int(col0),
            ws.buf.data_ptr(), ws.nbytes, flags, _stream(x2d.device))
    _lib.check(rc, "exl3_gemv_peers")
    exchange.pending = my_ctr
    if not defer_wait:
        exchange.settle(pdl=pdl)
    return view


def peer_allgather(y_local: torch.Tensor, *, exchange, cols_total: int, col0: int, pdl: bool = False,
                   defer_wait: bool = False) -> torch.Tensor:
    """(rows, local) slice -> this rank's complete (rows, cols_total) row, over peer memory.
    defer_wait as in gemv_peers."""
    _need_cuda(y_local, "y_local")
    rows, cols = y_local.shape
    if y_local.stride(1) != 1:
        y_local = y_local.contiguous()
    lib = _lib.load()
    exchange.settle(pdl=pdl)
    _, y_ptrs, c_ptrs, view, my_ctr = exchange.take(rows, cols_total)
    _lib.check(lib.exl3_peer_allgather(y_local.data_ptr(), rows, cols, y_local.stride(0), y_ptrs, c_ptrs,
                                       exchange.world, cols_total, int(col0), _flags(pdl), _stream(y_local.device)),
               "exl3_peer_allgather")
    exchange.pending = my_ctr
    if not defer_wait:
        exchange.settle(pdl=pdl)
    return view
