"""Host-side mirror of the reference's operator surface for the GGUF linear path, over the C ABI.

Names and argument meaning follow the ``Backend`` trait family of the reference (src/backend/mod.rs):
``prepare_weight`` (:333), ``linear`` (:389), ``linear_add`` (:417), ``dual_linear`` / ``triple_linear``
(:444-451), ``gated_linear`` (:467), ``gated_mlp`` / ``gated_mlp_add_residual`` (:474, :483), and the MoE
entry points (:1627-2025).  torch is used only for device memory and streams; every operator is a call into
``libzq_b200.so``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import ffi

_DTYPES = {torch.float32: ffi.F32, torch.float16: ffi.F16, torch.bfloat16: ffi.BF16}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported activation dtype {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class Weight:
    """Resident packed weight (``CudaWeight`` / ``CudaGgufPacked``, src/backend/cuda/resident.rs:82-107)."""

    def __init__(self, ctx: "B200Context", handle: C.c_void_p):
        self.ctx = ctx
        self.handle = handle

    @property
    def rows(self) -> int:
        return ffi.load().zq_weight_rows(self.handle)

    @property
    def cols(self) -> int:
        return ffi.load().zq_weight_cols(self.handle)

    @property
    def tensor_type(self) -> int:
        return ffi.load().zq_weight_type(self.handle)

    @property
    def gguf_bytes(self) -> int:
        return ffi.load().zq_weight_gguf_bytes(self.handle)

    def release(self):
        if self.handle:
            ffi.load().zq_weight_release(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class B200Context:
    """One device, one stream (``CudaContext``, src/backend/cuda/context.rs:248-276)."""

    def __init__(self, device: int = 0, use_torch_stream: bool = True):
        self.lib = ffi.load()
        handle = C.c_void_p()
        ffi.call("zq_ctx_create", device, C.byref(handle))
        self.handle = handle
        self.device = torch.device("cuda", device)
        if use_torch_stream:
            self.set_stream(torch.cuda.current_stream(self.device).cuda_stream)

    # ---- context
    def set_stream(self, cuda_stream: int):
        ffi.call("zq_ctx_set_stream", self.handle, C.c_void_p(cuda_stream))

    def sync(self):
        ffi.call("zq_ctx_sync", self.handle)

    def set_option(self, key: str, value: int):
        ffi.call("zq_ctx_set_option", self.handle, key.encode(), int(value))

    @property
    def sm_count(self) -> int:
        return self.lib.zq_ctx_sm_count(self.handle)

    @property
    def launch_count(self) -> int:
        return int(self.lib.zq_ctx_launch_count(self.handle))

    def close(self):
        if self.handle:
            self.lib.zq_ctx_destroy(self.handle)
            self.handle = None

    # ---- weights
    def prepare_weight(self, tensor_type: int, data, rows: int, cols: int) -> Weight:
        """``prepare_weight(LinearWeight::gguf)``: ``data`` is GGUF-layout bytes (bytes, numpy uint8 or a uint8 tensor)."""
        out = C.c_void_p()
        if isinstance(data, torch.Tensor) and data.is_cuda:
            data = data.contiguous()
            ffi.call("zq_weight_prepare_device", self.handle, tensor_type, _ptr(data), data.numel(), rows, cols, C.byref(out))
            self.sync()
        else:
            if isinstance(data, torch.Tensor):
                data = data.contiguous().numpy()
            buf = memoryview(data).cast("B")
            arr = (C.c_uint8 * len(buf)).from_buffer_copy(buf) if buf.readonly else (C.c_uint8 * len(buf)).from_buffer(buf)
            ffi.call("zq_weight_prepare", self.handle, tensor_type, arr, len(buf), rows, cols, C.byref(out))
        return Weight(self, out)

    def quantize(self, tensor_type: int, values: torch.Tensor) -> torch.Tensor:
        """f32 ``[rows, cols]`` on the device -> GGUF-layout bytes (uint8 tensor)."""
        values = values.contiguous().float()
        rows, cols = values.shape
        e, b = ffi.BLOCK[tensor_type]
        if cols % e:
            raise ffi.ZqFailure(1, f"columns {cols} not aligned to block {e}")
        out = torch.empty(rows * (cols // e) * b, dtype=torch.uint8, device=values.device)
        ffi.call("zq_quantize", self.handle, tensor_type, _ptr(values), rows, cols, _ptr(out), out.numel())
        return out

    def dequantize(self, w: Weight) -> torch.Tensor:
        out = torch.empty((w.rows, w.cols), dtype=torch.float32, device=self.device)
        ffi.call("zq_dequantize_f32", self.handle, w.handle, _ptr(out))
        return out

    def gather_rows(self, w: Weight, row_ids: Optional[torch.Tensor], n_rows: Optional[int] = None, dtype=torch.float16) -> torch.Tensor:
        n = int(row_ids.numel()) if row_ids is not None else int(n_rows)
        if row_ids is not None:
            row_ids = row_ids.to(device=self.device, dtype=torch.int32).contiguous()
        out = torch.empty((n, w.cols), dtype=dtype, device=self.device)
        ffi.call("zq_gather_rows", self.handle, w.handle, _ptr(row_ids), n, _ptr(out), _DTYPES[dtype])
        return out

    # ---- linear family
    def _rows(self, x: torch.Tensor, cols: int) -> int:
        if x.dim() == 1:
            x = x.unsqueeze(0)
        if x.shape[-1] != cols:
            raise ffi.ZqFailure(1, f"linear input cols={x.shape[-1]}, weight cols={cols}")
        return x.numel() // cols

    def linear(self, x: torch.Tensor, w: Weight, out_dtype=None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = x.contiguous()
        m = self._rows(x, w.cols)
        out_dtype = out_dtype or x.dtype
        y = torch.empty((m, w.rows), dtype=out_dtype, device=x.device)
        if residual is not None:
            residual = residual.contiguous()
            if residual.numel() != y.numel() or residual.dtype != out_dtype:
                raise ffi.ZqFailure(1, f"residual shape/dtype mismatch: {tuple(residual.shape)} {residual.dtype} vs {tuple(y.shape)} {out_dtype}")
        ffi.call("zq_linear", self.handle, w.handle, _ptr(x), _dt(x), m, _ptr(y), _DTYPES[out_dtype], _ptr(residual))
        return y

    def linear_add(self, x: torch.Tensor, w: Weight, residual: torch.Tensor, out_dtype=None) -> torch.Tensor:
        return self.linear(x, w, out_dtype=out_dtype or residual.dtype, residual=residual)

    def linear_batch(self, jobs, out_dtype=None):
        """Independent decode projections in as few launches as possible (``zq_linear_batch``).

        ``jobs`` is a list of ``(x, weight)``, ``(x, weight, residual)``, ``(x, gate, up, "gated")`` or
        ``(x, weight, residual_or_None, "row")`` tuples (the last form is a row-parallel job: its result is summed over the
        ranks of the peer group); all inputs share one dtype.  Returns the list of outputs."""
        arr = (ffi.ZqLinearJob * len(jobs))()
        ys, keep = [], []
        x_dt = None
        for i, job in enumerate(jobs):
            x = job[0].contiguous()
            gated = len(job) == 4 and job[3] == "gated"
            w = job[1]
            m = self._rows(x, w.cols)
            x_dt = x_dt or x.dtype
            if x.dtype != x_dt:
                raise TypeError("linear_batch: all inputs must share one dtype")
            od = out_dtype or x.dtype
            y = torch.empty((m, w.rows), dtype=od, device=x.device)
            row = len(job) == 4 and job[3] == "row"
            residual = job[2].contiguous() if ((len(job) == 3 or row) and job[2] is not None) else None
            arr[i].w = w.handle.value
            arr[i].w_up = job[2].handle.value if gated else None
            arr[i].dev_x = x.data_ptr()
            arr[i].m = m
            arr[i].dev_y = y.data_ptr()
            arr[i].dev_residual = residual.data_ptr() if residual is not None else None
            arr[i].flags = ffi.JOB_ROW_PARALLEL if row else 0
            ys.append(y)
            keep.append((x, residual))
        if jobs:
            ffi.call("zq_linear_batch", self.handle, arr, len(jobs), _DTYPES[x_dt], _DTYPES[out_dtype or x_dt])
        return ys

    def linear_row_parallel(self, x: torch.Tensor, w: Weight, out_dtype=None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """This rank's column slice of a weight against its slice of the input; the ranks' partial results are summed
        (``zq_linear_row_parallel``)."""
        x = x.contiguous()
        m = self._rows(x, w.cols)
        out_dtype = out_dtype or x.dtype
        y = torch.empty((m, w.rows), dtype=out_dtype, device=x.device)
        if residual is not None:
            residual = residual.contiguous()
        ffi.call("zq_linear_row_parallel", self.handle, w.handle, _ptr(x), _dt(x), m, _ptr(y), _DTYPES[out_dtype], _ptr(residual))
        return y

    def dist_init(self, slot_bytes: int = 4 << 20, group=None):
        """Joins the peer group of the node: allocates this rank's exchange buffer, exchanges the handles of all ranks
        through ``torch.distributed`` (any transport would do: the library only sees the bytes) and maps the peers."""
        import torch.distributed as dist

        world, rank = dist.get_world_size(group), dist.get_rank(group)
        blob = (C.c_uint8 * ffi.DIST_HANDLE_BYTES)()
        ffi.call("zq_dist_export", self.handle, int(slot_bytes), blob)
        ffi.call("zq_dist_init", self.handle, rank, world, self._exchange_blobs(blob, group))

    def _exchange_blobs(self, blob, group=None):
        import torch.distributed as dist

        world = dist.get_world_size(group)
        mine = torch.tensor(list(blob), dtype=torch.uint8, device=self.device if dist.get_backend(group) == "nccl" else "cpu")
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine, group=group)
        flat = bytes(torch.cat(gathered).cpu().tolist())
        return (C.c_uint8 * len(flat)).from_buffer_copy(flat)

    def moe_ep_init(self, max_tokens_per_rank: int, hidden: int, top_k: int, num_experts_total: int, dtype=torch.bfloat16, group=None):
        """Expert-parallel exchange buffers of this rank (after ``dist_init``): allocate, exchange handles, map the peers."""
        blob = (C.c_uint8 * ffi.DIST_HANDLE_BYTES)()
        ffi.call("zq_moe_ep_export", self.handle, int(max_tokens_per_rank), int(hidden), int(top_k), int(num_experts_total), _DTYPES[dtype], blob)
        ffi.call("zq_moe_ep_init", self.handle, self._exchange_blobs(blob, group))

    def linear_multi(self, x: torch.Tensor, weights: Sequence[Weight], out_dtype=None):
        x = x.contiguous()
        m = self._rows(x, weights[0].cols)
        out_dtype = out_dtype or x.dtype
        ys = [torch.empty((m, w.rows), dtype=out_dtype, device=x.device) for w in weights]
        wa = (C.c_void_p * len(weights))(*[w.handle for w in weights])
        ya = (C.c_void_p * len(weights))(*[y.data_ptr() for y in ys])
        ffi.call("zq_linear_multi", self.handle, wa, len(weights), _ptr(x), _dt(x), m, ya, _DTYPES[out_dtype])
        return ys

    def rmsnorm_linear_multi(self, x: torch.Tensor, norm_weight: torch.Tensor, eps: float, weights: Sequence[Weight], out_dtype=None, weight_offset: float = 0.0):
        """RMSNorm of every row, then the projections (``Backend::rmsnorm_linear`` / ``rmsnorm_dual_linear``,
        src/backend/mod.rs:455-464); ``weight_offset`` 1.0 is the Gemma form of the norm."""
        x = x.contiguous()
        m = self._rows(x, weights[0].cols)
        norm_weight = norm_weight.contiguous().float()
        if norm_weight.numel() != weights[0].cols:
            raise ffi.ZqFailure(1, f"norm weight has {norm_weight.numel()} elements, input width is {weights[0].cols}")
        out_dtype = out_dtype or x.dtype
        ys = [torch.empty((m, w.rows), dtype=out_dtype, device=x.device) for w in weights]
        wa = (C.c_void_p * len(weights))(*[w.handle for w in weights])
        ya = (C.c_void_p * len(weights))(*[y.data_ptr() for y in ys])
        ffi.call("zq_rmsnorm_linear", self.handle, wa, len(weights), _ptr(x), _dt(x), m, _ptr(norm_weight), float(eps), float(weight_offset), ya, _DTYPES[out_dtype])
        return ys

    def rmsnorm_linear(self, x, norm_weight, eps: float, w: Weight, out_dtype=None, weight_offset: float = 0.0):
        return self.rmsnorm_linear_multi(x, norm_weight, eps, [w], out_dtype, weight_offset)[0]

    def rmsnorm_dual_linear(self, x, norm_weight, eps: float, first: Weight, second: Weight, out_dtype=None, weight_offset: float = 0.0):
        a, b = self.rmsnorm_linear_multi(x, norm_weight, eps, [first, second], out_dtype, weight_offset)
        return a, b

    def dual_linear(self, x, first: Weight, second: Weight, out_dtype=None):
        a, b = self.linear_multi(x, [first, second], out_dtype)
        return a, b

    def triple_linear(self, x, first: Weight, second: Weight, third: Weight, out_dtype=None):
        a, b, c = self.linear_multi(x, [first, second, third], out_dtype)
        return a, b, c

    def rope_prefix_qk(self, query: torch.Tensor, key: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, rotary_dim: int, position: int, cos: torch.Tensor, sin: torch.Tensor,
                       interleaved: bool = False, suffix: bool = False):
        """``Backend::rope_prefix_qk`` (src/backend/mod.rs:567; ``suffix=True`` is ``rope``): rotates q and k in place,
        one launch; ``cos`` / ``sin`` are f32 device tables [positions, rotary_dim / 2]."""
        rows = query.shape[0] if query.dim() > 1 else 1
        head_dim = query.numel() // rows // num_heads
        if key is not None and (key.dtype != query.dtype or key.numel() != rows * num_kv_heads * head_dim):
            raise ffi.ZqFailure(1, "rope: key shape or dtype does not match the query's")
        cos, sin = cos.contiguous().float(), sin.contiguous().float()
        if cos.numel() != sin.numel():
            raise ffi.ZqFailure(1, f"rope: cos and sin tables differ in length ({cos.numel()} / {sin.numel()})")
        ffi.call("zq_rope_qk", self.handle, _ptr(query), num_heads, _ptr(key), num_kv_heads if key is not None else 0, _dt(query), rows, head_dim, rotary_dim, int(interleaved), int(suffix), position,
                 _ptr(cos), _ptr(sin), cos.numel())
        return query, key

    def gated_linear(self, x: torch.Tensor, gate: Weight, up: Weight, out_dtype=None) -> torch.Tensor:
        x = x.contiguous()
        m = self._rows(x, gate.cols)
        out_dtype = out_dtype or x.dtype
        y = torch.empty((m, gate.rows), dtype=out_dtype, device=x.device)
        ffi.call("zq_gated_silu", self.handle, gate.handle, up.handle, _ptr(x), _dt(x), m, _ptr(y), _DTYPES[out_dtype])
        return y

    def gated_mlp(self, x: torch.Tensor, gate: Weight, up: Weight, down: Weight, out_dtype=None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = x.contiguous()
        m = self._rows(x, gate.cols)
        out_dtype = out_dtype or x.dtype
        y = torch.empty((m, down.rows), dtype=out_dtype, device=x.device)
        if residual is not None:
            residual = residual.contiguous()
        ffi.call("zq_gated_mlp", self.handle, gate.handle, up.handle, down.handle, _ptr(x), _dt(x), m, _ptr(y), _DTYPES[out_dtype], _ptr(residual))
        return y

    def gated_mlp_add_residual(self, x, gate, up, down, residual, out_dtype=None):
        return self.gated_mlp(x, gate, up, down, out_dtype=out_dtype or residual.dtype, residual=residual)

    def begin_batch(self):
        """Backend::begin_batch: host-buffer calls until finish_batch are enqueued, not waited for."""
        ffi.call("zq_batch_begin", self.handle)

    def finish_batch(self):
        """Backend::finish_batch: waits once for everything enqueued since begin_batch and fills the output buffers."""
        ffi.call("zq_batch_finish", self.handle)

    def linear_host(self, x_host, w: Weight, y_host):
        """Host-buffer linear: numpy arrays in and out, copies inside the call."""
        import numpy as np

        dt = {np.dtype(np.float32): ffi.F32, np.dtype(np.float16): ffi.F16}
        m = x_host.size // w.cols
        ffi.call("zq_linear_host", self.handle, w.handle, C.c_void_p(x_host.ctypes.data), dt[x_host.dtype], m, C.c_void_p(y_host.ctypes.data), dt[y_host.dtype])
        return y_host


    def linear_host_batch(self, jobs):
        """A whole bracket in one call (``zq_linear_host_batch``): ``jobs`` is a list of ``(x_host, weight, y_host)`` numpy
        triples sharing one input dtype and one output dtype."""
        import numpy as np

        dt = {np.dtype(np.float32): ffi.F32, np.dtype(np.float16): ffi.F16}
        arr = (ffi.ZqLinearHostJob * len(jobs))()
        for i, (x_host, w, y_host) in enumerate(jobs):
            arr[i].w = w.handle.value
            arr[i].host_x = x_host.ctypes.data
            arr[i].m = x_host.size // w.cols
            arr[i].host_y = y_host.ctypes.data
        ffi.call("zq_linear_host_batch", self.handle, arr, len(jobs), dt[jobs[0][0].dtype], dt[jobs[0][2].dtype])


class GgufFile:
    """``GgufReader`` (src/weight/container/gguf.rs:332-566): header, metadata and tensor directory of a GGUF v3 file (or
    of a set of standard split files); matrices and expert slices go straight to resident weights."""

    def __init__(self, path: str):
        handle = C.c_void_p()
        ffi.call("zq_gguf_open", str(path).encode(), C.byref(handle))
        self.handle = handle

    def close(self):
        if self.handle:
            ffi.load().zq_gguf_close(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensor_names(self):
        out = []
        buf = C.create_string_buffer(512)
        for i in range(ffi.load().zq_gguf_tensor_count(self.handle)):
            ffi.call("zq_gguf_tensor_name", self.handle, i, buf, len(buf))
            out.append(buf.value.decode())
        return out

    def tensor_info(self, name: str):
        """``(type, dims in GGUF order, bytes)``"""
        t, nd, nb = C.c_uint32(), C.c_uint32(), C.c_uint64()
        dims = (C.c_uint64 * 4)()
        ffi.call("zq_gguf_tensor_info", self.handle, name.encode(), C.byref(t), C.byref(nd), dims, C.byref(nb))
        return t.value, [int(dims[i]) for i in range(nd.value)], int(nb.value)

    def metadata_u64(self, key: str) -> int:
        v = C.c_uint64()
        ffi.call("zq_gguf_metadata_u64", self.handle, key.encode(), C.byref(v))
        return int(v.value)

    def metadata_f64(self, key: str) -> float:
        v = C.c_double()
        ffi.call("zq_gguf_metadata_f64", self.handle, key.encode(), C.byref(v))
        return float(v.value)

    def metadata_str(self, key: str) -> str:
        buf = C.create_string_buffer(4096)
        ffi.call("zq_gguf_metadata_str", self.handle, key.encode(), buf, len(buf))
        return buf.value.decode()

    def load_matrix(self, ctx: "B200Context", name: str) -> Weight:
        out = C.c_void_p()
        ffi.call("zq_gguf_load_matrix", ctx.handle, self.handle, name.encode(), C.byref(out))
        return Weight(ctx, out)

    def load_matrix_slice(self, ctx: "B200Context", name: str, index: int) -> Weight:
        out = C.c_void_p()
        ffi.call("zq_gguf_load_matrix_slice", ctx.handle, self.handle, name.encode(), int(index), C.byref(out))
        return Weight(ctx, out)


def lm_head_argmax(ctx: B200Context, head: Weight, x: torch.Tensor) -> torch.Tensor:
    """Greedy token ids of an LM-head projection, computed on the device (``zq_lm_head_argmax``)."""
    x = x.contiguous()
    m = x.numel() // head.cols
    ids = torch.empty(m, dtype=torch.int32, device=x.device)
    ffi.call("zq_lm_head_argmax", ctx.handle, head.handle, _ptr(x), _dt(x), m, _ptr(ids))
    return ids


class MoeExperts:
    """Resident expert table (replaces ``CudaMoeState``'s cache when every expert fits in HBM,
    src/backend/cuda/expert.rs:284-570).  Keeps the weights alive for as long as the table."""

    def __init__(self, ctx: B200Context, gate: Sequence[Weight], up: Sequence[Weight], down: Sequence[Weight]):
        self.ctx, self.gate, self.up, self.down = ctx, list(gate), list(up), list(down)
        n = len(self.gate)
        ga = (C.c_void_p * n)(*[w.handle for w in self.gate])
        ua = (C.c_void_p * n)(*[w.handle for w in self.up])
        da = (C.c_void_p * n)(*[w.handle for w in self.down])
        out = C.c_void_p()
        ffi.call("zq_moe_experts_create", ctx.handle, ga, ua, da, n, C.byref(out))
        self.handle = out

    def __del__(self):
        try:
            if self.handle:
                ffi.load().zq_moe_experts_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


def moe_route(ctx: B200Context, x: torch.Tensor, router: torch.Tensor, top_k: int, scaling_factor: float = 1.0, normalize_selected: bool = True, bias: Optional[torch.Tensor] = None, scoring: int = ffi.ROUTE_SOFTMAX):
    """``moe_route_softmax_topk_device_f32`` (src/kernel/cuda/routing.rs:167) and, with ``scoring``, the bias-corrected
    routers of src/moe/routing.rs:43-81: returns ``(ids [m, k] int32, weights [m, k] f32)`` on the device."""
    x = x.contiguous()
    router = router.contiguous().float()
    m, hidden = x.shape
    experts = router.shape[0]
    ids = torch.empty((m, top_k), dtype=torch.int32, device=x.device)
    w = torch.empty((m, top_k), dtype=torch.float32, device=x.device)
    ffi.call("zq_moe_route_topk", ctx.handle, int(scoring), _ptr(x), _dt(x), m, hidden, _ptr(router), _ptr(bias), experts, top_k, float(scaling_factor), int(normalize_selected), _ptr(ids), _ptr(w))
    return ids, w


def moe_gather_rows(ctx: B200Context, x: torch.Tensor, row_ids: torch.Tensor) -> torch.Tensor:
    """``Backend::moe_gather_rows`` (src/backend/mod.rs:1657): ``out[i] = x[row_ids[i]]``."""
    x = x.contiguous()
    row_ids = row_ids.to(device=x.device, dtype=torch.int32).contiguous()
    out = torch.empty((row_ids.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    ffi.call("zq_moe_gather_rows", ctx.handle, _ptr(x), _dt(x), x.shape[0], x.shape[1], _ptr(row_ids), row_ids.numel(), _ptr(out))
    return out


def moe_scatter_add_rows(ctx: B200Context, accumulator: torch.Tensor, rows: torch.Tensor, row_ids: torch.Tensor, weights: Optional[torch.Tensor]) -> torch.Tensor:
    """``Backend::moe_scatter_add_rows`` (src/backend/mod.rs:1661): ``accumulator[row_ids[i]] += weights[i] * rows[i]`` (f32 accumulator, in place)."""
    rows = rows.contiguous()
    row_ids = row_ids.to(device=rows.device, dtype=torch.int32).contiguous()
    if weights is not None:
        weights = weights.contiguous().float()
    if accumulator.dtype != torch.float32 or not accumulator.is_contiguous():
        raise TypeError("the MoE accumulator is a contiguous f32 tensor")
    ffi.call("zq_moe_scatter_add_rows", ctx.handle, _ptr(rows), _dt(rows), _ptr(row_ids), _ptr(weights), rows.shape[0], rows.shape[1], _ptr(accumulator), accumulator.shape[0])
    return accumulator


def moe_forward_ep(ctx: B200Context, local_experts: MoeExperts, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, shared=None, residual: Optional[torch.Tensor] = None, out_dtype=None,
                   max_tokens_any_rank: int = 0) -> torch.Tensor:
    """Expert-parallel routed experts (``zq_moe_forward_ep``): ``local_experts`` are this rank's block of the experts,
    ``ids`` are global expert ids of this rank's own tokens; ``max_tokens_any_rank`` is the largest token count of any
    rank in this call (0: all ranks bring as many tokens as this one)."""
    x = x.contiguous()
    m, hidden = x.shape
    out_dtype = out_dtype or x.dtype
    y = torch.empty((m, hidden), dtype=out_dtype, device=x.device)
    ids = ids.contiguous()
    weights = weights.contiguous().float()
    top_k = ids.numel() // m
    sg, su, sd = (w.handle for w in shared) if shared is not None else (None, None, None)
    if residual is not None:
        residual = residual.contiguous()
    ffi.call("zq_moe_forward_ep", ctx.handle, local_experts.handle, sg, su, sd, _ptr(x), _dt(x), m, int(max_tokens_any_rank), _ptr(ids), _ptr(weights), top_k, _ptr(y), _DTYPES[out_dtype], _ptr(residual))
    return y


def moe_forward(ctx: B200Context, experts: MoeExperts, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, shared=None, residual: Optional[torch.Tensor] = None, out_dtype=None) -> torch.Tensor:
    """Routed experts (+ shared expert, + residual): ``prefill_resident_routed_experts_add`` / ``decode_routed_experts``
    (src/backend/mod.rs:1921-1960, 2012-2024).  ``shared`` is ``(gate, up, down)`` or None."""
    x = x.contiguous()
    m, hidden = x.shape
    out_dtype = out_dtype or x.dtype
    y = torch.empty((m, hidden), dtype=out_dtype, device=x.device)
    ids = ids.contiguous()
    weights = weights.contiguous().float()
    top_k = ids.numel() // m
    sg, su, sd = (w.handle for w in shared) if shared is not None else (None, None, None)
    if residual is not None:
        residual = residual.contiguous()
    ffi.call("zq_moe_forward", ctx.handle, experts.handle, sg, su, sd, _ptr(x), _dt(x), m, _ptr(ids), _ptr(weights), top_k, _ptr(y), _DTYPES[out_dtype], _ptr(residual))
    return y
