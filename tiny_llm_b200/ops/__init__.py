"""Python face of the sm_100a kernels.  Every op checks its tensors, picks the kernel for the
dtype and sizes, and launches it on torch's current stream through the C entry points of the
shared objects that `build.py` compiles from csrc/.  There is no other path: an op given a tensor
that is not on a CUDA device, or called where the kernels cannot be built, raises."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build
from .build import BuildError

F32, BF16 = 0, 1
OUT_SAME, OUT_F32, OUT_ACC = 0, 1, 2


class KernelError(RuntimeError):
    """A kernel refused its arguments (a size it is not built for) or failed to launch."""


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    # torch's current stream of the current device as a raw cudaStream_t (the private accessor is
    # an order of magnitude cheaper than building a Stream object for every launch)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the engine's ops run on a CUDA device only; got a tensor on " + str(t.device))


launches = 0  # kernels launched through this module since import (each entry point launches one)
_pdl = True


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch: each kernel is launched so that its prologue (and, for the
    matrix products, its first weight tiles) may overlap the tail of the kernel before it."""
    global _pdl
    _pdl = bool(on)
    for lib in build._loaded.values():
        lib.tllm_set_pdl(1 if _pdl else 0)


_tape = None   # while a list: every launch is also noted there as (library, function, arguments), see begin_tape()


def _call(lib, fn, *args):
    """Calls one entry point of a compiled library (one kernel launch, or a few) and raises its message if it refuses."""
    global launches
    if fn(*args) != 0:
        raise KernelError(lib.tllm_last_error().decode())
    launches += 1
    if _tape is not None:
        _tape.append((lib, fn, args))


def begin_tape() -> None:
    """From here to end_tape() the launches are noted as they are made: the compiled functions with the very argument
    objects they got.  A step whose launches depend on nothing but what the caller knows (the sizes of the step and the
    addresses of buffers that stay where they are) can be run again from such a tape without walking the model's
    Python code: the step's tables are read by the kernels from device memory, as in a captured graph."""
    global _tape
    _tape = []


def end_tape():
    global _tape
    tape, _tape = _tape, None
    return tape


def replay_tape(tape) -> None:
    global launches
    for lib, fn, args in tape:
        if fn(*args) != 0:
            raise KernelError(lib.tllm_last_error().decode())
    launches += len(tape)


def knobs():
    """The module's switches that decide which kernels a step launches; a tape or graph holds for one setting of them."""
    return (force_generic, split_k, cluster_mask, attention_tc, decode_wide_ctas, decode_cluster_merge, qkv_fused_rows,
            linear_skinny, generic_attention_split, split_mixed_attention, _pdl)


def _i32(t: Optional[torch.Tensor], name: str):
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{name} must be a contiguous int32 tensor")


def trace_dump():
    """The timeline notes of every loaded library since the last call (needs a TLLM_TRACE=1 build):
    a list of (t_enter ns, t_ready ns, grid x, y, z, block x, library, marks), sorted by t_enter.  t_ready
    of a launch is when the kernel before it in the stream had finished; marks are up to four more
    moments a kernel noted itself (0: none)."""
    import struct
    out = []
    buf = ctypes.create_string_buffer(8192 * 64)
    for key, lib in build._loaded.items():
        if not hasattr(lib, "tllm_trace_dump"):
            continue
        n = lib.tllm_trace_dump(buf, 8192)
        for i in range(n):
            t0, t1, gx, gy, gz, bx, m0, m1, m2, m3 = struct.unpack_from("<QQIIIIQQQQ", buf, i * 64)
            out.append((t0, t1, gx, gy, gz, bx, key, (m0, m1, m2, m3)))
    return sorted(out)


# ----------------------------------------------------------------------------- elementwise


def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :] = table[tokens[t], :] as float32 (the residual stream is 32-bit)."""
    _need_cuda(tokens, table, out)
    _i32(tokens, "tokens")
    t, h = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous() or table.shape[1] != h \
            or tokens.numel() != t:
        raise KernelError("embedding: shapes or dtypes do not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_embedding, _ptr(tokens), _ptr(table), _ptr(out), t, h, _code(table.dtype), _stream())


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
             rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = weight * x[rows[r], :] / sqrt(mean(x^2) + eps); x and weight are float32."""
    _need_cuda(x, weight, out, rows)
    _i32(rows, "rows")
    h = x.shape[1]
    n = out.shape[0]
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or not x.is_contiguous() or \
            not out.is_contiguous() or out.shape[1] != h or weight.numel() != h or \
            (rows is None and n != x.shape[0]) or (rows is not None and rows.numel() != n):
        raise KernelError("rms_norm: shapes or dtypes do not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_rms_norm, _ptr(x), _ptr(weight), _ptr(out), _ptr(rows), n, h, ctypes.c_float(eps),
                                  _code(out.dtype), _stream())


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, block: int, consume: bool = False) -> None:
    """out[m, g*block + j] = silu(gate_up[m, 2*g*block + j]) * gate_up[m, 2*g*block + block + j].
    consume=True: `gate_up` is a float32 accumulation buffer (split-K sums) and is handed back zeroed."""
    _need_cuda(gate_up, out)
    m, inter = out.shape
    if gate_up.shape != (m, 2 * inter) or not gate_up.is_contiguous() or not out.is_contiguous() or \
            (consume and gate_up.dtype != torch.float32) or (not consume and gate_up.dtype != out.dtype):
        raise KernelError("silu_mul: shapes or dtypes do not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_silu_mul, _ptr(gate_up), _ptr(out), m, inter, block, _code(gate_up.dtype), _code(out.dtype),
                                  1 if consume else 0, _stream())


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, cos: Optional[torch.Tensor],
                  sin: Optional[torch.Tensor], rot_dim: int, num_heads: int, num_kv_heads: int, head_dim: int,
                  k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  slot_mapping: Optional[torch.Tensor], src: Optional[torch.Tensor] = None) -> None:
    """Rotates the queries of `qkv` in place; rotates the keys and writes keys and values into the
    pages at slot_mapping (None: the row holds queries only and nothing is written).
    `src`: float32 rows to read instead of `qkv` (a split-K accumulation buffer, handed back zeroed);
    the rotated queries still go to `qkv`."""
    _need_cuda(qkv, positions, cos, sin, k_cache, v_cache, slot_mapping, src)
    if src is not None and (src.dtype != torch.float32 or src.shape != qkv.shape or src.stride(1) != 1):
        raise KernelError("rope_kv_write: the float32 source must have the shape of qkv")
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    t, width = qkv.shape
    want = num_heads * head_dim + (0 if slot_mapping is None else 2 * num_kv_heads * head_dim)
    if width != want or qkv.stride(1) != 1:
        raise KernelError(f"rope_kv_write: rows of {width} values, expected {want}")
    page_size = page_stride = head_stride = 0
    if slot_mapping is not None:
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype or k_cache.shape != v_cache.shape or \
                k_cache.stride() != v_cache.stride() or k_cache.stride(3) != 1 or k_cache.stride(2) != head_dim:
            raise KernelError("rope_kv_write: cache layout does not fit")
        page_size, page_stride, head_stride = k_cache.shape[2], k_cache.stride(0), k_cache.stride(1)
    if cos is not None and (cos.dtype != torch.float32 or not cos.is_contiguous() or cos.shape[1] * 2 != rot_dim):
        raise KernelError("rope_kv_write: rotary tables do not fit")
    lib = build.load_library("elementwise")
    _call(lib, lib.tllm_rope_kv_write,
        _ptr(qkv), _ptr(src), 0 if src is None else src.stride(0), _ptr(positions), _ptr(cos), _ptr(sin), rot_dim, t,
        num_heads, num_kv_heads, head_dim,
        qkv.stride(0), _ptr(k_cache if slot_mapping is not None else None),
        _ptr(v_cache if slot_mapping is not None else None), _ptr(slot_mapping), page_size,
        ctypes.c_longlong(page_stride), ctypes.c_longlong(head_stride), _code(qkv.dtype), _stream())


# ----------------------------------------------------------------------------- matrix products


EPI_BF16, EPI_F32, EPI_ADD_F32, EPI_SWIGLU, EPI_ATOMIC_F32 = 0, 1, 2, 3, 4
EPI_CL_ADD_F32, EPI_CL_ROPE_KV, EPI_CL_SWIGLU, EPI_CL_BF16 = 5, 6, 7, 8   # K slices reduced inside a thread-block cluster
_sm_count = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (cudaDevAttrMultiProcessorCount), read once per device:
    the slice counts below are sized to fill them."""
    index = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if index not in _sm_count:
        _sm_count[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_count[index]


force_generic = False   # tests set this to compare the tensor-core kernels with the SIMT ones
split_k = os.environ.get("TLLM_SPLIT_K", "1") != "0"   # slices of K at decode (a switch for measurements)
# which products of few rows reduce their K slices inside a thread-block cluster instead of with float32
# atomics: 1 = residual add / plain store, 2 = Q/K/V with rotation and cache write, 4 = SiLU * up.
# Measured at the TinyLlama shape (decode, batch 8): 0 -> 1.109 ms, 6 -> 1.087 ms, 7 -> 1.185 ms per
# step: the fused epilogues save a kernel each, the cluster's barriers cost about as much as one.
cluster_mask = int(os.environ.get("TLLM_CLUSTER", "6"))
cluster_reduce = cluster_mask != 0
_status = {}


def status_word(device) -> torch.Tensor:
    """The device int in which a kernel records that one of its bounded waits expired."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


_STATUS_CODES = ("1 = TMA producer, 2 = MMA issuer, 3 = epilogue of a matrix product; 7 = TMA producer, "
                 "8 = MMA issuer, 9 = softmax of the tensor-core attention")


def raise_status(device, code: int) -> None:
    """Clears the device's status word and raises for the code that was read from it."""
    key = torch.device(device).index or 0
    if key in _status:
        _status[key].zero_()
    raise KernelError(f"a kernel on device {key} gave up waiting (code {code}: {_STATUS_CODES}); "
                      f"the step's output is not valid and was dropped")


def check_status() -> None:
    """Reads the status words (a device synchronisation) and raises if a kernel gave up a wait.
    The generation path does not call this: there the word travels with the sampled ids
    (`argmax` / `sample` with `status`)."""
    for key, t in _status.items():
        code = int(t.item())
        if code:
            raise_status(f"cuda:{key}", code)


def _tc_ok(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    k = a.shape[1]
    return (not force_generic and a.dtype == torch.bfloat16 and k % 8 == 0 and a.stride(0) % 8 == 0 and
            a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _swap_splits(n: int, k: int, atomic_ok: bool) -> int:
    """How many slices of K a weight tile of 128 rows is cut into at decode: enough CTAs to have
    every SM stream weights, but at least four 64-wide blocks per slice.  (Measured: counts that fill
    the SMs more evenly but with fewer CTAs -- 9 instead of 10 slices of the down projection, 3 instead
    of 2 for gate/up -- made the step slower, not faster.)"""
    if not atomic_ok or not split_k:
        return 1
    row_tiles = -(-n // 128)
    k_blocks = -(-k // 64)
    want = -(-sm_count() // row_tiles)
    return max(1, min(want, k_blocks // 4))


def _cluster_slices(n: int, k: int, limit: int = 8) -> int:
    """Slices of K per weight tile for the cluster kernel: 1, 2, 4 or 8, enough CTAs for every SM, at
    least four 64-wide blocks per slice."""
    s = _swap_splits(n, k, True)
    p = 1
    while p * 2 <= min(s, limit):
        p *= 2
    return p


def _cluster_call(epi, a, w, out, slices, positions=None, cos=None, sin=None, nq=0, nkv=0, hd=0, k_cache=None,
                  v_cache=None, slot_mapping=None):
    lib = build.load_library("linear_tc")
    m, k = a.shape
    page_size = page_stride = head_stride = 0
    if k_cache is not None:
        page_size, page_stride, head_stride = k_cache.shape[2], k_cache.stride(0), k_cache.stride(1)
    _call(lib, lib.tllm_linear_tc_cluster,
        _ptr(a), _ptr(w), _ptr(out), m, w.shape[0], k, a.stride(0), out.stride(0), epi, slices, _ptr(positions),
        _ptr(cos), _ptr(sin), nq, nkv, hd, _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping), page_size,
        ctypes.c_longlong(page_stride), ctypes.c_longlong(head_stride), _ptr(status_word(a.device)), _stream())


def linear_rope_kv(h: torch.Tensor, w_qkv: torch.Tensor, qkv: torch.Tensor, positions: torch.Tensor,
                   cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                   head_dim: int, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                   slot_mapping: Optional[torch.Tensor]) -> bool:
    """Q/K/V projection with the rotation and the cache write in its epilogue (a cluster per weight tile
    for at most 128 tokens, 128 x 256 tiles of the product for more):
    the rotated queries go to the first num_heads*head_dim values of each `qkv` row, rotated keys and
    values straight into their pages (slot_mapping None: `w_qkv` holds the query rows only).  Returns
    False, having done nothing, where the fused kernel does not apply (then: linear + rope_kv_write)."""
    m = h.shape[0]
    if not ((cluster_mask & 2) and _tc_ok(h, w_qkv, qkv) and head_dim in ((16, 32, 64, 128) if m <= 128 else (64, 128)) and
            qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and w_qkv.is_contiguous() and
            (cos is None or cos.shape[1] * 2 == head_dim)):
        return False
    _need_cuda(h, w_qkv, qkv, positions, cos, sin, k_cache, v_cache, slot_mapping)
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    want = num_heads * head_dim + (0 if slot_mapping is None else 2 * num_kv_heads * head_dim)
    if w_qkv.shape != (want, h.shape[1]) or qkv.shape[0] != m or qkv.shape[1] < num_heads * head_dim:
        raise KernelError("linear_rope_kv: shapes do not fit")
    if slot_mapping is not None and (k_cache.dtype != torch.bfloat16 or k_cache.stride() != v_cache.stride() or
                                     k_cache.stride(3) != 1 or k_cache.stride(2) != head_dim):
        raise KernelError("linear_rope_kv: cache layout does not fit")
    _cluster_call(EPI_CL_ROPE_KV, h, w_qkv, qkv, _cluster_slices(want, h.shape[1]) if m <= 128 else 1, positions, cos, sin, num_heads,
                  num_kv_heads, head_dim, k_cache if slot_mapping is not None else None,
                  v_cache if slot_mapping is not None else None, slot_mapping)
    return True


# Up to this many tokens (and above 128, where the product runs as 128 x 256 tiles) the Q/K/V projection takes the
# kernel with rotation and cache write in its epilogue, whatever the sizes.  Between, a cluster of eight K slices hands
# round 8 x 128 x tokens float32 values per weight tile, and K slices added with float32 atomics plus the
# rotate-and-cache kernel are faster (ms per decode step at the TinyLlama sizes, 8 slices, fused / separate: 16 tokens
# 0.935 / 0.932, 24 1.059 / 1.063, 32 1.123 / 1.097, 64 1.576 / 1.518); with fewer slices the fused kernel stays
# (Llama-3-8B sizes, 4 slices, 8 layers: 32 tokens 1.326 / 1.428, 64 1.802 / 1.840).
qkv_fused_rows = int(os.environ.get("TLLM_QKV_FUSED_ROWS", "24"))


def fused_qkv_preferred(m: int, n: int, k: int) -> bool:
    return m <= qkv_fused_rows or m > 128 or _cluster_slices(n, k) < 8


# float32 products of at most 16 rows take a kernel of their own (one thread per output element, weights streamed
# through shared memory); False keeps the 64 x 64 tiles.  Both give the same bits (tests compare them).
linear_skinny = True


def prefers_split(a: torch.Tensor, w: torch.Tensor) -> bool:
    """True when `linear` would cut K into slices for this product if it may add into a float32
    output: few rows (decode), so few weight tiles that the SMs only fill when K is split too.
    A caller that wants a bfloat16 result then accumulates into a zeroed float32 buffer and lets the
    next kernel convert (silu_mul / rope_kv_write with consume/src)."""
    return _tc_ok(a, w, None) and a.shape[0] <= 128 and _swap_splits(w.shape[0], a.shape[1], True) > 1


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out = a . w^T (w is [N, K], rows contiguous).  `out` may be of a's dtype or float32;
    accumulate=True adds the product into a float32 `out`.  bfloat16 products run on the tensor
    cores (tcgen05) when K and the row stride of `a` are multiples of 8; float32 products, and
    the sizes TMA cannot take, run on the SIMT kernel."""
    _need_cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n) or a.dtype != w.dtype or a.stride(1) != 1 or \
            out.stride(1) != 1 or not w.is_contiguous():
        raise KernelError(f"linear: shapes or dtypes do not fit: a {tuple(a.shape)} {a.dtype}, "
                          f"w {tuple(w.shape)} {w.dtype}, out {tuple(out.shape)} {out.dtype}")
    if accumulate:
        if out.dtype != torch.float32:
            raise KernelError("linear: accumulation needs a float32 output")
        mode = OUT_ACC
    elif out.dtype == a.dtype:
        mode = OUT_SAME
    elif out.dtype == torch.float32:
        mode = OUT_F32
    else:
        raise KernelError(f"linear: output dtype {out.dtype} does not fit input dtype {a.dtype}")
    if _tc_ok(a, w, out):
        lib = build.load_library("linear_tc")
        epi = {OUT_SAME: EPI_BF16, OUT_F32: EPI_F32, OUT_ACC: EPI_ADD_F32}[mode]
        swap, splits = 0, 1
        if m <= 128:
            swap = 1
            if (cluster_mask & 1) and mode in (OUT_ACC, OUT_SAME):
                slices = _cluster_slices(n, k)
                if slices > 1:   # the slices of K meet in a cluster: one writer per element, no atomics
                    _cluster_call(EPI_CL_ADD_F32 if mode == OUT_ACC else EPI_CL_BF16, a, w, out, slices)
                    return
            splits = _swap_splits(n, k, atomic_ok=(mode == OUT_ACC))
            if splits > 1:
                epi = EPI_ATOMIC_F32
        _call(lib, lib.tllm_linear_tc, _ptr(a), _ptr(w), _ptr(out), m, n, k, a.stride(0), out.stride(0), epi, swap,
                                       splits, _ptr(status_word(a.device)), _stream())
        return
    lib = build.load_library("linear_generic")
    _call(lib, lib.tllm_linear_generic, _ptr(a), _ptr(w), _ptr(out), m, n, k, a.stride(0), out.stride(0),
                                        _code(a.dtype), mode, int(linear_skinny), _stream())


def linear_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, block: int, workspace) -> None:
    """out = silu(a Wg^T) * (a Wu^T) with Wg, Wu interleaved in `w_gate_up` in row blocks of `block`.
    With blocks of 128 and more than 128 rows the product and SiLU*up are one tensor-core kernel."""
    m = a.shape[0]
    n2 = w_gate_up.shape[0]
    if _tc_ok(a, w_gate_up, out) and block == 128 and m > 128 and n2 % 256 == 0 and out.is_contiguous():
        _need_cuda(a, w_gate_up, out)
        lib = build.load_library("linear_tc")
        _call(lib, lib.tllm_linear_tc, _ptr(a), _ptr(w_gate_up), _ptr(out), m, n2, a.shape[1], a.stride(0),
                                       out.stride(0), EPI_SWIGLU, 0, 1, _ptr(status_word(a.device)), _stream())
        return
    if (cluster_mask & 4) and _tc_ok(a, w_gate_up, out) and block == 128 and m <= 128 and n2 % 256 == 0 and \
            out.stride(1) == 1 and w_gate_up.is_contiguous():
        # the gate tile, the up tile beside it and their K slices form one cluster; SiLU * up in its epilogue
        _need_cuda(a, w_gate_up, out)
        _cluster_call(EPI_CL_SWIGLU, a, w_gate_up, out, _cluster_slices(n2, a.shape[1], limit=4))
        return
    if prefers_split(a, w_gate_up):
        acc = workspace.get_zeroed("gate_up_f32", (m, n2))
        linear(a, w_gate_up, acc, accumulate=True)
        silu_mul(acc, out, block, consume=True)
        return
    gu = workspace.get("gate_up", (m, n2), a.dtype)
    linear(a, w_gate_up, gu)
    silu_mul(gu, out, block)


# ----------------------------------------------------------------------------- attention


attention_tc = os.environ.get("TLLM_ATTENTION_TC", "1") != "0"   # tcgen05 attention for prompt portions (a switch for measurements)


def _attention_splits(num_requests: int, max_q_len: int, group: int, num_kv_heads: int, max_kv_len: int) -> int:
    """Slices of keys per (request, key/value head).  Decoded tokens (at most 16 rows) run as small
    CTAs: the fewest slices that give at least 256 CTAs of at most 11 tiles of 64 keys each, each slice
    at least two tiles, and no slice empty.  (Measured at context 2,048: batch 1 -> 16 slices, 8 -> 8,
    16 -> 4, 32 and 64 -> 3; "fill three CTAs per SM once" had picked 14 at batch 8 and 2 at batch 64 and
    was 5 to 7 % slower.)  Portions of prompts are sliced only when there are fewer CTAs than SMs."""
    if max_q_len * group <= 16:
        ctas = num_requests * num_kv_heads
        tiles = max(1, -(-max_kv_len // 64))
        most = max(1, tiles // 2)
        pick = most
        for s in range(1, most + 1):
            if ctas * s >= 256 and -(-tiles // s) <= 11:
                pick = s
                break
        per_slice = -(-tiles // pick)
        return -(-tiles // per_slice)
    ctas = num_requests * (-(-max_q_len * group // 64)) * num_kv_heads
    sms = sm_count()
    if ctas >= sms:
        return 1
    return max(1, min(-(-2 * sms // ctas), max_kv_len // 256))


# Decoded tokens with one warp per 64-key tile (slices of four tiles, all of a slice's copies in flight at once, one
# block barrier instead of one per tile): taken when it gives this many CTAs.  Measured at the TinyLlama sizes,
# context 2,048, against the kernel that walks a slice tile by tile with four warps per tile (ms per step): batch 4
# 0.754 / 0.778, 8 0.810 / 0.826, 16 0.938 / 0.942; outside the range it loses: batch 1 0.724 / 0.716 (32 CTAs),
# batch 32 1.193 / 1.124 (1,024 CTAs).  TLLM_DECODE_WIDE=0 turns it off (a switch for measurements).
decode_wide_ctas = (96, 640) if os.environ.get("TLLM_DECODE_WIDE", "1") != "0" else (1, 0)
# ... and its 2 to 8 slices of a (request, key/value head) as one thread-block cluster that merges them over
# distributed shared memory, in place of partial results in global memory and a merging kernel behind it, while the
# CTAs are at most 1.75 per SM: a cluster starts only when all its CTAs find room at once, and past that count whole
# clusters wait for a second round (ms per step with / without, context 2,048: batch 4 0.744 / 0.753, 6 0.774 / 0.777,
# 8 0.800 / 0.811, but 9 0.871 / 0.829, 12 0.931 / 0.872, 16 0.973 / 0.940; the kernel that walks a slice tile by tile
# gains nothing from it at any batch: 64 1.547 / 1.506, 32 1.080 / 1.085, 24 1.084 / 1.063).  TLLM_DECODE_CLUSTER=0 turns it off.
decode_cluster_merge = os.environ.get("TLLM_DECODE_CLUSTER", "1") != "0"


def _cluster_merge(num_requests: int, num_kv_heads: int, splits: int) -> bool:
    return decode_cluster_merge and 2 <= splits <= 8 and num_requests * num_kv_heads * splits * 4 <= 7 * sm_count()


def _wide_splits(num_requests: int, num_kv_heads: int, max_kv_len: int) -> int:
    """Slices of four tiles for the kernel with one warp per tile, or 0 where it is not taken."""
    splits = -(-max(1, -(-max_kv_len // 64)) // 4)
    lo, hi = decode_wide_ctas
    ctas = num_requests * num_kv_heads * splits
    if lo <= ctas <= hi:
        return splits
    # fewer CTAs than that: only where the slices then merge inside a cluster, which saves the merge kernel
    # (batch 1 at context 2,048: 0.684 ms per step against 0.714, batch 2 0.707 against 0.732)
    return splits if ctas < lo and hi > 0 and _cluster_merge(num_requests, num_kv_heads, splits) else 0


# The attention of the 32-bit path runs eight warps per (token, head) or one warp per (token, key/value head, four query
# heads), by the number of pairs; both give the same bits.  True / False force one of them, 2 the plainest form (one
# warp per pair); tests compare the three.
generic_attention_split = None


split_mixed_attention = os.environ.get("TLLM_SPLIT_MIXED_ATTENTION", "1") != "0"   # (a switch for measurements)


class _SubBatch:
    """Requests [lo, hi) of a step's batch, for a kernel that takes a run of the per-request tables."""

    def __init__(self, batch, lo: int, hi: int, max_q_len: int):
        self.cu_q = batch.cu_q[lo: hi + 1]
        self.q_start = batch.q_start[lo: hi]
        self.num_requests = hi - lo
        self.max_q_len = max_q_len
        self.max_kv_len = batch.max_kv_len
        self.token_request = batch.token_request
        self.positions = batch.positions
        self.num_leading_decodes = 0


def paged_attention(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, k_cache: torch.Tensor,
                    v_cache: torch.Tensor, block_table: torch.Tensor, batch, out: torch.Tensor, scale: float,
                    window: Optional[int] = None, workspace=None) -> None:
    """Attention of every token of the step (queries in the first num_heads*head_dim values of each
    `qkv` row) over its request's pages.  `batch` carries the step's metadata: token_request and
    positions per token; cu_q, q_start per request; num_requests, max_q_len, max_kv_len.
    bfloat16 runs on the tensor-core kernel compiled for this head size (it needs `workspace` for the
    partial results when it slices the keys); float32 on the SIMT kernel."""
    _need_cuda(qkv, k_cache, v_cache, block_table, out)
    _i32(block_table, "block_table")
    t = qkv.shape[0]
    if out.shape != (t, num_heads * head_dim) or not out.is_contiguous() or out.dtype != qkv.dtype or \
            k_cache.dtype != qkv.dtype or k_cache.stride() != v_cache.stride() or k_cache.stride(3) != 1 or \
            k_cache.stride(2) != head_dim or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
        raise KernelError("paged_attention: shapes or dtypes do not fit")
    page_size = k_cache.shape[2]
    group = num_heads // num_kv_heads
    if qkv.dtype == torch.bfloat16 and not force_generic and attention_tc and head_dim in ATTENTION_TC_HEAD_DIMS and \
            not window and batch.max_q_len * group >= 128 and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0 and \
            k_cache.is_contiguous() and v_cache.is_contiguous():
        # portions of prompts: 128 rows of (token, head of the group) per CTA on the tcgen05 tensor cores
        lib = build.load_library("attention_tc", flags=(f"-DTLLM_HEAD_DIM={head_dim}",))
        if lib.tllm_attention_tc_fits(num_heads, num_kv_heads, head_dim, page_size, 0):
            lead = getattr(batch, "num_leading_decodes", 0)
            if 0 < lead < batch.num_requests and group <= 16 and split_mixed_attention:
                # Decoded tokens beside portions, the decoded ones first (as the scheduler lays a step out): a CTA of
                # 128 rows would walk a whole context for the one token of a request.  They go to the decode kernel,
                # the rest to this one: two launches over two runs of the same tables.
                paged_attention(qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache, block_table[:lead],
                                _SubBatch(batch, 0, lead, 1), out, scale, window, workspace)
                paged_attention(qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache, block_table[lead:],
                                _SubBatch(batch, lead, batch.num_requests, batch.max_q_len), out, scale, window, workspace)
                return
            _call(lib, lib.tllm_attention_tc,
                _ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), ctypes.c_longlong(k_cache.shape[0]),
                _ptr(block_table), block_table.shape[1], _ptr(batch.cu_q), _ptr(batch.q_start), _ptr(out), t,
                batch.num_requests, batch.max_q_len, num_heads, num_kv_heads, head_dim, page_size,
                ctypes.c_float(scale), _ptr(status_word(qkv.device)), _stream())
            return
    if qkv.dtype == torch.bfloat16 and not force_generic and head_dim % 16 == 0 and 16 <= head_dim <= 256 and \
            qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0:
        lib = build.load_library("attention_mma", flags=(f"-DTLLM_HEAD_DIM={head_dim}",))
        splits, wide = 1, 0   # wide: bit 0 = one warp per tile, bit 1 = the slices merge inside a cluster
        if workspace is not None:
            splits = _attention_splits(batch.num_requests, batch.max_q_len, group, num_kv_heads, batch.max_kv_len)
            if batch.max_q_len * group <= 16:
                wide_splits = _wide_splits(batch.num_requests, num_kv_heads, batch.max_kv_len) \
                    if lib.tllm_attention_mma_wide_fits() else 0
                if wide_splits:
                    splits, wide = wide_splits, (3 if _cluster_merge(batch.num_requests, num_kv_heads, wide_splits) else 1)
        scratch = None
        if splits > 1 and not wide & 2:
            scratch = workspace.get("attention_partials", (t * num_heads * splits * (head_dim + 2),), torch.float32)
        _call(lib, lib.tllm_attention_mma,
            _ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
            _ptr(batch.cu_q), _ptr(batch.q_start), _ptr(out), t, batch.num_requests, batch.max_q_len, num_heads,
            num_kv_heads, head_dim, page_size, ctypes.c_longlong(k_cache.stride(0)),
            ctypes.c_longlong(k_cache.stride(1)), ctypes.c_float(scale), int(window or 0), splits, _ptr(scratch),
            wide, int(batch.max_kv_len), _stream())
        return
    lib = build.load_library("attention_generic")
    _call(lib, lib.tllm_paged_attention_generic,
        _ptr(qkv), qkv.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(batch.token_request), _ptr(batch.positions), _ptr(out), t, num_heads, num_kv_heads, head_dim,
        page_size, ctypes.c_longlong(k_cache.stride(0)), ctypes.c_longlong(k_cache.stride(1)),
        ctypes.c_float(scale), int(window or 0), _code(qkv.dtype),
        -1 if generic_attention_split is None else int(generic_attention_split), _stream())


def attention_tc_timing(head_dim: int = 64) -> Optional[dict]:
    """Cycles that the roles of the prompt-attention kernel's first CTA spent per phase since the last call, or
    None if the kernel was not built with TLLM_NVCC_FLAGS_ATTENTION_TC=-DTLLM_ATT_TIMING=1."""
    if head_dim not in ATTENTION_TC_HEAD_DIMS:
        return None
    lib = build.load_library("attention_tc", flags=(f"-DTLLM_HEAD_DIM={head_dim}",))
    if not hasattr(lib, "tllm_attention_tc_timing"):
        return None
    out = (ctypes.c_ulonglong * 16)()
    lib.tllm_attention_tc_timing(out)
    names = ["softmax: wait S", "softmax: S to registers", "softmax: max, exp2, sum", "softmax: P to tensor memory",
             "(unused)", "softmax: vote, store wait", "softmax: fence, arrive", "rescales of O",
             "qk: wait K", "qk: wait S buffer", "pv: wait V", "qk: issue", "tma: wait free stage", "tma: issue",
             "pv: wait P", "pv: issue"]
    return {n: int(v) for n, v in zip(names, out) if n != "(unused)"}


# ----------------------------------------------------------------------------- sampling


def argmax(logits: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """out[i] = first maximum of row i.  `status`: the device's status word; `out` then holds n + 1
    ints and out[n] receives the word, so that it travels to the host with the ids."""
    _need_cuda(logits, out, status)
    _i32(out, "out")
    _i32(status, "status")
    n, v = logits.shape
    if logits.dtype != torch.float32 or not logits.is_contiguous() or out.numel() != n + (status is not None):
        raise KernelError("argmax: logits must be contiguous float32 [n, V] and out int32 [n] (n + 1 with a status word)")
    lib = build.load_library("sampling")
    _call(lib, lib.tllm_argmax, _ptr(logits), _ptr(out), n, v, _ptr(status), _stream())


def sample(logits: torch.Tensor, work: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor, out: torch.Tensor,
           status: Optional[torch.Tensor] = None) -> None:
    """Temperature -> top-k -> top-p -> multinomial per row; rows with temperature <= 0 are greedy.
    `work` is float32 scratch of at least n*V elements; seeds and counters are int64 (read as
    unsigned 64-bit).  `status` as for argmax."""
    _need_cuda(logits, work, temperature, top_k, top_p, seeds, counters, out, status)
    _i32(top_k, "top_k")
    _i32(out, "out")
    _i32(status, "status")
    n, v = logits.shape
    if logits.dtype != torch.float32 or not logits.is_contiguous() or work.dtype != torch.float32 or \
            work.numel() < n * v or temperature.dtype != torch.float32 or top_p.dtype != torch.float32 or \
            seeds.dtype != torch.int64 or counters.dtype != torch.int64 or out.numel() != n + (status is not None) or \
            any(x.numel() != n for x in (temperature, top_k, top_p, seeds, counters)):
        raise KernelError("sample: shapes or dtypes do not fit")
    lib = build.load_library("sampling")
    _call(lib, lib.tllm_sample, _ptr(logits), _ptr(work), n, v, _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                _ptr(seeds), _ptr(counters), _ptr(out), _ptr(status), _stream())


ALL_LIBRARIES = ("elementwise", "linear_generic", "linear_tc", "attention_generic", "sampling")


ATTENTION_HEAD_DIMS = (16, 32, 48, 64, 128)   # head sizes `build_all` compiles ahead; others compile on first use
ATTENTION_TC_HEAD_DIMS = (64, 128)            # head sizes the tcgen05 prompt-attention kernel is written for


def build_all(verbose: bool = True):
    """Compiles every library (what `__graft_entry__.build()` calls); returns their paths."""
    paths = [build.compile_library(n, verbose=verbose) for n in ALL_LIBRARIES]
    paths += [build.compile_library("attention_mma", flags=(f"-DTLLM_HEAD_DIM={hd}",), verbose=verbose)
              for hd in ATTENTION_HEAD_DIMS]
    paths += [build.compile_library("attention_tc", flags=(f"-DTLLM_HEAD_DIM={hd}",), verbose=verbose)
              for hd in ATTENTION_TC_HEAD_DIMS]
    return paths
