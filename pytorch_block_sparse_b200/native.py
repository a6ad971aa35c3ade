"""ctypes binding of libbsmm_b200.so (declared in ``include/bsmm_b200.h``) plus the thin
torch-facing helpers the matrix class uses.  torch only supplies device memory and the
current stream here; every byte of arithmetic happens in the library's CUDA kernels.

There is no CPU path: a missing library or a non-CUDA tensor raises.
"""
import ctypes
import os

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libbsmm_b200.so")

# mirrors include/bsmm_b200.h
ABI_VERSION = 2
OK = 0
PREC_FP32_SIMT, PREC_TF32X3, PREC_BF16, PREC_TF32, PREC_BF16X3 = 0, 1, 2, 3, 4
DSD_DGRAD, DSD_OUT_COLMAJOR, DSD_GELU, DSD_IO_BF16 = 0x10, 0x20, 0x40, 0x80
SDDMM_A_COLMAJOR, SDDMM_B_COLMAJOR, SDDMM_IO_BF16 = 0x10, 0x20, 0x40

PRECISIONS = {"fp32": PREC_FP32_SIMT, "simt": PREC_FP32_SIMT, "tf32x3": PREC_TF32X3, "tf32": PREC_TF32, "bf16": PREC_BF16,
              "bf16x3": PREC_BF16X3}
EXPORTS = (
    "bsmm_abi_version",
    "bsmm_status_string",
    "bsmm_last_cuda_error",
    "bsmm_device_status",
    "bsmm_debug_trace_dsd",
    "bsmm_packed_bytes",
    "bsmm_pack_weights",
    "bsmm_plan_group",
    "bsmm_plan_bytes",
    "bsmm_build_plan",
    "bsmm_dsd",
    "bsmm_dsd_fused",
    "bsmm_dsd_multi",
    "bsmm_dsd_scatter",
    "bsmm_sum_row_slots",
    "bsmm_allreduce_peers",
    "bsmm_sddmm_plan_bytes",
    "bsmm_build_sddmm_plan",
    "bsmm_sddmm_workspace_bytes",
    "bsmm_sddmm",
    "bsmm_sddmm_static",
    "bsmm_rebuild_indices",
    "bsmm_select_lowest",
    "bsmm_sample_free_cells",
    "bsmm_move_blocks",
)

_lib = None
_default_precision = os.environ.get("BSMM_PRECISION", "tf32x3")


class NativeError(RuntimeError):
    pass


def load():
    """dlopen the library once and declare the argument types of every export."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise NativeError(
            "%s is missing: build it with `python -m pytorch_block_sparse_b200.build` "
            "(this package has no CPU or PyTorch fallback)" % LIB_PATH
        )
    lib = ctypes.CDLL(LIB_PATH)
    c = ctypes
    vp, i64, u32, i32 = c.c_void_p, c.c_int64, c.c_uint32, c.c_int
    lib.bsmm_abi_version.restype = i32
    lib.bsmm_abi_version.argtypes = []
    lib.bsmm_status_string.restype = c.c_char_p
    lib.bsmm_status_string.argtypes = [i32]
    lib.bsmm_last_cuda_error.restype = i32
    lib.bsmm_last_cuda_error.argtypes = []
    lib.bsmm_device_status.restype = i32
    lib.bsmm_device_status.argtypes = [c.POINTER(c.c_uint), i32]
    lib.bsmm_debug_trace_dsd.restype = i32
    lib.bsmm_debug_trace_dsd.argtypes = [vp, i32]
    lib.bsmm_packed_bytes.restype = i64
    lib.bsmm_packed_bytes.argtypes = [i64, u32]
    lib.bsmm_pack_weights.restype = i32
    lib.bsmm_pack_weights.argtypes = [vp, i64, u32, vp, vp, vp]
    lib.bsmm_plan_group.restype = i32
    lib.bsmm_plan_group.argtypes = [i64, i64, i64, u32]
    lib.bsmm_plan_bytes.restype = i64
    lib.bsmm_plan_bytes.argtypes = [i64, i64, i32]
    lib.bsmm_build_plan.restype = i32
    lib.bsmm_build_plan.argtypes = [vp, vp, i64, i64, i32, vp, vp]
    lib.bsmm_dsd.restype = i32
    lib.bsmm_dsd.argtypes = [vp, i64, i64, vp, vp, i64, vp, vp, vp, i64, vp, vp, u32, vp]
    lib.bsmm_dsd_fused.restype = i32
    lib.bsmm_dsd_fused.argtypes = [vp, i64, i64, vp, vp, i64, vp, vp, vp, i64, vp, vp, vp, vp, u32, vp]
    lib.bsmm_dsd_multi.restype = i32
    lib.bsmm_dsd_multi.argtypes = [vp, i64, i64, vp, vp, i64, vp, vp, vp, i64, vp, i64, i64, vp, vp, vp, vp, i32, u32, vp]
    lib.bsmm_dsd_scatter.restype = i32
    lib.bsmm_dsd_scatter.argtypes = [vp, i64, i64, vp, vp, i64, vp, vp, vp, i64, vp, vp, i32, i32, u32, vp]
    lib.bsmm_sum_row_slots.restype = i32
    lib.bsmm_sum_row_slots.argtypes = [vp, i32, i64, i64, vp, i32, i64, vp]
    lib.bsmm_allreduce_peers.restype = i32
    lib.bsmm_allreduce_peers.argtypes = [vp, i32, i32, i64, ctypes.c_float, vp]
    lib.bsmm_sddmm_workspace_bytes.restype = i64
    lib.bsmm_sddmm_workspace_bytes.argtypes = [i64, i64, i64, i64, u32]
    lib.bsmm_sddmm.restype = i32
    lib.bsmm_sddmm.argtypes = [vp, vp, i64, i64, i64, vp, vp, i64, vp, vp, vp, vp, u32, vp]
    lib.bsmm_sddmm_static.restype = i32
    lib.bsmm_sddmm_static.argtypes = [vp, vp, i64, i64, i64, vp, vp, i64, vp, vp, vp, u32, vp]
    lib.bsmm_sddmm_plan_bytes.restype = i64
    lib.bsmm_sddmm_plan_bytes.argtypes = [i64, i64]
    lib.bsmm_build_sddmm_plan.restype = i32
    lib.bsmm_build_sddmm_plan.argtypes = [vp, i64, i64, vp, vp]
    lib.bsmm_rebuild_indices.restype = i32
    lib.bsmm_rebuild_indices.argtypes = [vp, i64, i64, i64, vp, vp, vp, vp, vp, vp, vp]
    lib.bsmm_select_lowest.restype = i32
    lib.bsmm_select_lowest.argtypes = [vp, i64, i64, vp, vp]
    lib.bsmm_sample_free_cells.restype = i32
    lib.bsmm_sample_free_cells.argtypes = [vp, i64, i64, i64, c.c_uint64, vp, vp, vp, vp]
    lib.bsmm_move_blocks.restype = i32
    lib.bsmm_move_blocks.argtypes = [vp, vp, vp, i64, i64, i64, vp, vp]
    if lib.bsmm_abi_version() != ABI_VERSION:
        raise NativeError("libbsmm_b200.so has ABI %d, this package expects %d" % (lib.bsmm_abi_version(), ABI_VERSION))
    _lib = lib
    return lib


def check(status, what):
    if status != OK:
        lib = load()
        msg = lib.bsmm_status_string(status).decode()
        extra = ""
        if status == 3:
            extra = " [cudaError_t=%d]" % lib.bsmm_last_cuda_error()
        raise NativeError("%s failed: %s%s" % (what, msg, extra))


def device_status(clear=True):
    """Device health word (synchronizes): non-zero after a kernel abandoned a bounded wait."""
    lib = load()
    word = ctypes.c_uint(0)
    check(lib.bsmm_device_status(ctypes.byref(word), 1 if clear else 0), "bsmm_device_status")
    return word.value


def set_default_precision(name):
    """'tf32x3' (default; fp32-class accuracy on tensor cores), 'bf16x3' (fp32-class too, about 5e-6 instead of
    2e-6: forward and input gradient add three products of bf16 hi and lo parts, half the tensor-core
    instructions; the weight gradient computes as 'tf32x3'), 'fp32' (CUDA-core FMA), 'tf32' (single
    tensor-core pass, the accuracy class of cuBLAS with allow_tf32) or 'bf16' (operands rounded to bf16 inside
    the kernels, fp32 tensors and accumulation)."""
    global _default_precision
    if name not in PRECISIONS:
        raise ValueError("unknown precision %r, expected one of %s" % (name, sorted(PRECISIONS)))
    _default_precision = name


def default_precision():
    """Name of the precision used when a call names none."""
    return _default_precision


def resolve_precision(precision):
    name = _default_precision if precision is None else precision
    if name not in PRECISIONS:
        raise ValueError("unknown precision %r, expected one of %s" % (name, sorted(PRECISIONS)))
    return PRECISIONS[name]


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _aligned(t, alignment=16):
    """``t`` itself when its storage pointer is aligned, else a copy with the same strides.  Torch allocations are
    512-byte aligned, but views are not, nor are the parameters and buffers of ``nn.DataParallel`` replicas
    (slices of one flat broadcast buffer: an int32 buffer after one with an odd element count sits on a 4-byte
    boundary), while the kernels read with 8- and 16-byte accesses and TMA wants 16-byte bases."""
    if t is None or t.data_ptr() % alignment == 0:
        return t
    return t.clone(memory_format=torch.preserve_format)


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _need_cuda(t, name):
    if not t.is_cuda:
        raise NativeError("%s must be a CUDA tensor (got %s); there is no CPU path" % (name, t.device))


class PackedWeights:
    """Kernel-ready images of one ``data`` tensor + the fused per-slot sum of squares."""

    def __init__(self, data, precision, images, block_sumsq):
        self.data = data
        self.precision = precision
        self.images = images
        self.block_sumsq = block_sumsq


def pack_weights(data, precision):
    """Run ``bsmm_pack_weights`` on ``data`` (fp32 ``[nnz*32, 32]``)."""
    _need_cuda(data, "data")
    lib = load()
    nnz = data.shape[0] // 32
    raw = _aligned(data.detach())
    sumsq = torch.empty(nnz, dtype=torch.float32, device=data.device)
    nbytes = lib.bsmm_packed_bytes(nnz, precision)
    images = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=data.device) if nbytes > 0 else None
    with torch.cuda.device(data.device):
        check(
            lib.bsmm_pack_weights(_ptr(raw), nnz, precision, _ptr(images), _ptr(sumsq), _stream(data.device)),
            "bsmm_pack_weights",
        )
    return PackedWeights(raw, precision, images, sumsq)


def block_sumsq(data):
    """Per-slot sum of squares of ``data`` (fp32 ``[nnz*32, 32]``) from the library's statistic kernel
    (``bsmm_pack_weights`` asked for no images)."""
    _need_cuda(data, "data")
    lib = load()
    nnz = data.shape[0] // 32
    raw = data.detach()
    if not raw.is_contiguous():
        raw = raw.contiguous()
    raw = _aligned(raw)
    sumsq = torch.empty(nnz, dtype=torch.float32, device=data.device)
    with torch.cuda.device(data.device):
        check(lib.bsmm_pack_weights(_ptr(raw), nnz, PREC_FP32_SIMT, None, _ptr(sumsq), _stream(data.device)),
              "bsmm_pack_weights")
    return sumsq


def rebuild_indices(blocks, n_block_rows, n_block_cols, cell_slot, row_ptr, cols_a, col_ptr, rows_b, status):
    """``bsmm_rebuild_indices``: CSR / CSC buffers (written in place) from the slot-order ``blocks`` list."""
    _need_cuda(blocks, "blocks")
    lib = load()
    with torch.cuda.device(blocks.device):
        check(
            lib.bsmm_rebuild_indices(
                _ptr(blocks), blocks.shape[0] // 2, n_block_rows, n_block_cols, _ptr(cell_slot), _ptr(row_ptr),
                _ptr(cols_a), _ptr(col_ptr), _ptr(rows_b), _ptr(status), _stream(blocks.device),
            ),
            "bsmm_rebuild_indices",
        )


def select_lowest(stat, k):
    """``bsmm_select_lowest``: int32 ``[k]`` indices of the ``k`` smallest entries of the fp32 vector ``stat``."""
    _need_cuda(stat, "stat")
    lib = load()
    stat = stat.detach().contiguous()
    out = torch.empty(k, dtype=torch.int32, device=stat.device)
    with torch.cuda.device(stat.device):
        check(lib.bsmm_select_lowest(_ptr(stat), stat.shape[0], k, _ptr(out), _stream(stat.device)), "bsmm_select_lowest")
    return out


def sample_free_cells(cell_slot, n_free, k, seed, status):
    """``bsmm_sample_free_cells``: int32 ``[k]`` distinct empty positions of ``cell_slot``, a function of the seed."""
    _need_cuda(cell_slot, "cell_slot")
    lib = load()
    scratch = torch.empty(max(n_free, 1), dtype=torch.int32, device=cell_slot.device)
    out = torch.empty(k, dtype=torch.int32, device=cell_slot.device)
    with torch.cuda.device(cell_slot.device):
        check(
            lib.bsmm_sample_free_cells(
                _ptr(cell_slot), cell_slot.numel(), n_free, k, ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF), _ptr(scratch),
                _ptr(out), _ptr(status), _stream(cell_slot.device),
            ),
            "bsmm_sample_free_cells",
        )
    return out


def move_blocks(blocks, slots, cells, n_block_cols, status):
    """``bsmm_move_blocks``: ``blocks[slots[j]]`` becomes position ``cells[j]`` (in place)."""
    lib = load()
    with torch.cuda.device(blocks.device):
        check(
            lib.bsmm_move_blocks(
                _ptr(blocks), _ptr(slots), _ptr(cells), slots.shape[0], n_block_cols, blocks.shape[0] // 2, _ptr(status),
                _stream(blocks.device),
            ),
            "bsmm_move_blocks",
        )


class DsdPlan:
    """Launch plans of the tensor-core dsd kernel for one (offsets, indices) pair, one per group size
    (the kernel's tile is 128 tokens x group*32 columns; the group is chosen from the token count)."""

    def __init__(self, ptr, idx):
        _need_cuda(ptr, "ptr")
        load()
        self.ptr = _aligned(ptr)
        self.idx = _aligned(idx)
        self.n_out_blocks = ptr.shape[0] - 1
        self.nnz = idx.shape[0]
        self._buffers = {}

    def group_for(self, m, precision):
        forced = os.environ.get("BSMM_PLAN_GROUP")
        if forced:
            return min(int(forced), 6) if precision in (PREC_TF32X3, PREC_BF16X3) else int(forced)
        return load().bsmm_plan_group(m, self.n_out_blocks, self.nnz, precision)

    def buffer(self, group):
        buf = self._buffers.get(group)
        if buf is None:
            lib = load()
            nbytes = lib.bsmm_plan_bytes(self.n_out_blocks, self.nnz, group)
            if nbytes < 0:
                raise NativeError("invalid plan group %r" % (group,))
            buf = torch.empty(nbytes, dtype=torch.uint8, device=self.ptr.device)
            with torch.cuda.device(self.ptr.device):
                check(
                    lib.bsmm_build_plan(
                        _ptr(self.ptr), _ptr(self.idx), self.n_out_blocks, self.nnz, group, _ptr(buf),
                        _stream(self.ptr.device),
                    ),
                    "bsmm_build_plan",
                )
            self._buffers[group] = buf
        return buf


def dsd_matmul(a, plan, packed, n_out, transpose, bias=None, out=None, out_colmajor=False, residual=None,
               activation=None, pre_activation=None, out_col0=0, peer_outs=()):
    """``a @ W.T (+bias)`` (``transpose=True``) or ``a @ W`` through ``bsmm_dsd``.  ``a``: contiguous ``[m, k]``.

    Forward only, tensor-core precisions: ``residual`` (``[m, n_out]``) is added with the bias,
    ``activation="gelu"`` is applied to the sum, and ``pre_activation`` (an ``[m, n_out]`` tensor to fill)
    receives the sum before the activation -- all inside the kernel's epilogue (``bsmm_dsd_fused``).

    ``out`` may be wider than ``n_out`` (``[m, width]``): the call then writes the column slice starting at
    ``out_col0``, and ``peer_outs`` (device pointers, as integers, of tensors laid out like ``out`` -- other GPUs'
    copies reached through peer mappings) receive the same slice tile by tile (``bsmm_dsd_multi``)."""
    _need_cuda(a, "dense_a")
    lib = load()
    m, k = a.shape
    prec = packed.precision
    # fp32 tensors in and out ('bf16' precision then rounds the operands inside the kernel) -- except that the 'bf16'
    # precision takes a bf16 activation tensor as it is and then also writes a bf16 output: half the bytes
    io16 = (a.dtype == torch.bfloat16 and prec == PREC_BF16 and not out_colmajor and residual is None
            and pre_activation is None and plan.nnz > 0 and k > 0)
    want = torch.bfloat16 if io16 else torch.float32
    if a.dtype != want:
        a = a.to(want)
    a = _aligned(a)
    if out is not None and out.dtype != want:
        raise NativeError("out must be %s for this call, got %s" % (want, out.dtype))
    if out is None:
        out = torch.empty((n_out, m) if out_colmajor else (m, n_out), dtype=want, device=a.device)
    out_ld = 0
    if not out_colmajor and out.dim() == 2 and out.shape[1] != n_out:
        out_ld = out.shape[1]
        if not out.is_contiguous() or out.shape[0] != m:
            raise NativeError("a wider out must be a contiguous [m, width] tensor")
    peer_array = (ctypes.c_void_p * max(1, len(peer_outs)))(*[ctypes.c_void_p(int(ptr)) for ptr in peer_outs])
    if activation not in (None, "gelu"):
        raise ValueError("unknown activation %r (None or 'gelu')" % (activation,))
    flags = prec | (0 if transpose else DSD_DGRAD) | (DSD_OUT_COLMAJOR if out_colmajor else 0)
    flags |= DSD_GELU if activation == "gelu" else 0
    flags |= DSD_IO_BF16 if io16 else 0
    plan_buf = None
    if prec != PREC_FP32_SIMT:
        group = plan.group_for(m, prec)
        plan_buf = plan.buffer(group)
        flags |= group << 8
    if bias is not None and bias.dtype != torch.float32:
        bias = bias.float()
    bias = _aligned(bias.detach()) if bias is not None else None
    if residual is not None:
        residual = _aligned(residual.detach().reshape(m, n_out).to(torch.float32).contiguous())
    if pre_activation is not None and (pre_activation.dtype != torch.float32 or not pre_activation.is_contiguous()
                                       or pre_activation.numel() != m * n_out):
        raise NativeError("pre_activation must be a contiguous float32 tensor of the output's size")
    with torch.cuda.device(a.device):
        check(
            lib.bsmm_dsd_multi(
                _ptr(a), m, k, _ptr(plan.ptr), _ptr(plan.idx), plan.nnz, _ptr(packed.data), _ptr(packed.images),
                _ptr(plan_buf), n_out, _ptr(out), out_ld, out_col0, _ptr(bias),
                _ptr(residual), _ptr(pre_activation), peer_array if peer_outs else None, len(peer_outs), flags,
                _stream(a.device),
            ),
            "bsmm_dsd",
        )
    return out


def dsd_scatter(a, plan, packed, n_out, transpose, parts, slot, scratch=None):
    """``a @ W.T`` or ``a @ W`` fused with a reduce-scatter over rows (``bsmm_dsd_scatter``): ``parts`` are the
    device pointers (integers) of every rank's ``[world, m / world, n_out]`` fp32 tensor of parts in rank order, own
    included; every completed tile is stored into slot ``slot`` (this rank's index) of the tensor of the rank
    owning the tile's rows.  ``scratch``: an ``[m, n_out]`` fp32 tensor (allocated when missing)."""
    _need_cuda(a, "dense_a")
    lib = load()
    m, k = a.shape
    prec = packed.precision
    if prec == PREC_FP32_SIMT:
        raise NativeError("the fused reduce-scatter needs a tensor-core precision")
    if a.dtype != torch.float32:
        a = a.float()
    if scratch is None:
        scratch = torch.empty((m, n_out), dtype=torch.float32, device=a.device)
    group = plan.group_for(m, prec)
    flags = prec | (0 if transpose else DSD_DGRAD) | (group << 8)
    part_array = (ctypes.c_void_p * len(parts))(*[ctypes.c_void_p(int(ptr)) for ptr in parts])
    with torch.cuda.device(a.device):
        check(
            lib.bsmm_dsd_scatter(
                _ptr(a), m, k, _ptr(plan.ptr), _ptr(plan.idx), plan.nnz, _ptr(packed.data), _ptr(packed.images),
                _ptr(plan.buffer(group)), n_out, _ptr(scratch), part_array, len(parts), slot, flags, _stream(a.device),
            ),
            "bsmm_dsd_scatter",
        )
    return scratch


def sum_row_slots(parts, outs, out_row0):
    """``outs[j][out_row0 : out_row0 + rows] = parts.sum(0)`` for every pointer in ``outs`` (``bsmm_sum_row_slots``):
    ``parts`` is this rank's ``[slots, rows, cols]`` fp32 tensor, ``outs`` device pointers (integers) of ``[*, cols]``
    fp32 tensors -- every rank's full tensor, the peers' through NVLink mappings."""
    _need_cuda(parts, "parts")
    lib = load()
    slots, rows, cols = parts.shape
    out_array = (ctypes.c_void_p * len(outs))(*[ctypes.c_void_p(int(ptr)) for ptr in outs])
    with torch.cuda.device(parts.device):
        check(
            lib.bsmm_sum_row_slots(_ptr(parts), slots, rows, cols, out_array, len(outs), out_row0, _stream(parts.device)),
            "bsmm_sum_row_slots",
        )


def allreduce_peers(bufs, rank, elems, scale, device):
    """In-place sum (times ``scale``) over the ranks' buffers ``bufs`` (device pointers as integers, rank order, own
    included) through peer mappings (``bsmm_allreduce_peers``); the caller synchronises the ranks around it."""
    lib = load()
    arr = (ctypes.c_void_p * len(bufs))(*[ctypes.c_void_p(int(ptr)) for ptr in bufs])
    with torch.cuda.device(device):
        check(lib.bsmm_allreduce_peers(arr, len(bufs), rank, elems, ctypes.c_float(scale), _stream(device)),
              "bsmm_allreduce_peers")


class SddmmPlan:
    """Item table of the tensor-core SDDMM kernel for one CSR (offsets, indices) pair."""

    def __init__(self, ptr, idx):
        _need_cuda(ptr, "ptr")
        lib = load()
        self.ptr = ptr = _aligned(ptr)
        self.idx = _aligned(idx)
        n_rows = ptr.shape[0] - 1
        nnz = idx.shape[0]
        self.buffer = torch.empty(lib.bsmm_sddmm_plan_bytes(n_rows, nnz), dtype=torch.uint8, device=ptr.device)
        with torch.cuda.device(ptr.device):
            check(
                lib.bsmm_build_sddmm_plan(_ptr(ptr), n_rows, nnz, _ptr(self.buffer), _stream(ptr.device)),
                "bsmm_build_sddmm_plan",
            )


SDDMM_STATIC_MAX_BYTES = 64 << 20


def sddmm_static(a, b, blocks, out, plan, block_sumsq=None, precision=None):
    """``bsmm_sddmm_static``: the weight gradient for callers that may not allocate device memory (stream
    capture in progress, a runtime that owns all device memory, allocator callbacks).  The token-range
    partial sums go to a scratch array inside the library image instead of a torch-allocated workspace;
    this wrapper itself allocates nothing, so it cannot convert its arguments either: ``a`` (dY
    ``[tokens, rows]``) and ``b`` (X ``[tokens, cols]``) must be contiguous fp32 CUDA tensors, ``out`` contiguous
    fp32, ``blocks`` int32 -- anything else raises.  Problems whose scratch need exceeds
    ``SDDMM_STATIC_MAX_BYTES`` are refused.  Calls that overlap on the GPU share the array and race; make the
    first call per device outside any capture."""
    _need_cuda(a, "dense_a")
    _need_cuda(b, "dense_b")
    for name, t, dtype in (("dense_a", a, torch.float32), ("dense_b", b, torch.float32), ("out", out, torch.float32),
                           ("blocks", blocks, torch.int32)):
        if t.dtype != dtype or not t.is_contiguous() or not t.is_cuda:
            raise NativeError("%s must be a contiguous %s CUDA tensor (got %s, contiguous=%s, %s)"
                              % (name, dtype, t.dtype, t.is_contiguous(), t.device))
    if block_sumsq is not None and (block_sumsq.dtype != torch.float32 or not block_sumsq.is_contiguous()):
        raise NativeError("block_sumsq must be a contiguous float32 tensor")
    if a.dim() != 2 or b.dim() != 2 or a.shape[0] != b.shape[0]:
        raise NativeError("dense_a and dense_b must be [tokens, rows] and [tokens, cols]")
    lib = load()
    prec = resolve_precision(precision) if not isinstance(precision, int) else precision
    tokens, rows = a.shape
    cols = b.shape[1]
    nnz = blocks.shape[0] // 2
    with torch.cuda.device(a.device):
        check(
            lib.bsmm_sddmm_static(
                _ptr(a), _ptr(b), rows, cols, tokens, _ptr(out), _ptr(blocks), nnz, _ptr(plan.idx), _ptr(plan.buffer),
                _ptr(block_sumsq), prec, _stream(a.device),
            ),
            "bsmm_sddmm_static",
        )
    return out


def sddmm(a, a_rowmajor, b, b_rowmajor, blocks, out, precision=None, block_sumsq=None, plan=None):
    """``out[s] = (a.T @ b)[block s]`` in ``data`` layout through ``bsmm_sddmm``.

    ``a``: dY ``[tokens, rows]``, ``b``: X ``[tokens, cols]``; ``*_rowmajor`` False means the tensor's
    transpose is the contiguous one.  ``plan`` (:class:`SddmmPlan`) enables the tensor-core kernel."""
    _need_cuda(a, "dense_a")
    lib = load()
    prec = resolve_precision(precision) if not isinstance(precision, int) else precision
    tokens, rows = a.shape
    cols = b.shape[1]
    nnz = blocks.shape[0] // 2
    io16 = (a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and prec == PREC_BF16 and a_rowmajor and b_rowmajor
            and plan is not None and tokens >= 32)
    if not io16 and (a.dtype != torch.float32 or b.dtype != torch.float32):
        a, b = a.float(), b.float()
    a, b, blocks = _aligned(a), _aligned(b), _aligned(blocks)
    flags = prec | (0 if a_rowmajor else SDDMM_A_COLMAJOR) | (0 if b_rowmajor else SDDMM_B_COLMAJOR)
    flags |= SDDMM_IO_BF16 if io16 else 0
    ws_bytes = lib.bsmm_sddmm_workspace_bytes(rows, cols, tokens, nnz, flags) if plan is not None else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device) if ws_bytes > 0 else None
    with torch.cuda.device(a.device):
        check(
            lib.bsmm_sddmm(
                _ptr(a), _ptr(b), rows, cols, tokens, _ptr(out), _ptr(blocks), nnz,
                _ptr(plan.idx) if plan is not None else None, _ptr(plan.buffer) if plan is not None else None,
                _ptr(block_sumsq), _ptr(ws), flags, _stream(a.device),
            ),
            "bsmm_sddmm",
        )
    return out
