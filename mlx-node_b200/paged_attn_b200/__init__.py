"""ctypes binding of libpaged_attn_b200.so (the C ABI in include/paged_attn_b200.h).

This module is a thin host-side mirror used by the tests and the benchmark; the
product is the shared library.  There is no fallback of any kind: if the
library is missing or a call fails, an exception is raised.

Device memory is passed as raw pointers.  Any object with a ``data_ptr()``
method (a torch tensor) or a plain ``int`` address is accepted.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "libpaged_attn_b200.so")

PA_OK = 0
STATUS_NAMES = {
    0: "PA_OK", 1: "PA_ERR_INVALID_ARG", 2: "PA_ERR_UNSUPPORTED", 3: "PA_ERR_OOM",
    4: "PA_ERR_OUT_OF_RANGE", 5: "PA_ERR_TIMEOUT", 6: "PA_ERR_CUDA", 7: "PA_ERR_NCCL",
}

# Every symbol include/paged_attn_b200.h declares.
EXPORTED_SYMBOLS = [
    "pa_last_error_string", "pa_version",
    "mlx_paged_attn_create_cache", "mlx_paged_attn_free_cache",
    "mlx_paged_attn_get_key_cache", "mlx_paged_attn_get_value_cache",
    "mlx_paged_attn_reshape_and_cache", "mlx_paged_attn_forward", "mlx_paged_attn_copy_blocks",
    "pa_array_from_device", "pa_array_from_host", "pa_array_data", "mlx_array_ndim",
    "mlx_array_shape", "mlx_array_dtype", "mlx_array_delete", "pa_set_device", "pa_set_stream",
    "pa_cache_create", "pa_cache_wrap", "pa_cache_free", "pa_cache_key_ptr", "pa_cache_value_ptr",
    "pa_cache_get_config", "pa_cache_check_errors", "pa_reshape_and_cache", "pa_copy_blocks",
    "pa_qk_norm_rope_and_cache", "pa_cache_create_fp8", "pa_cache_wrap_fp8", "pa_cache_is_fp8",
    "pa_cache_set_kv_scales", "pa_cache_get_kv_scales", "pa_cache_fp8_set_exact_decode",
    "pa_gather_heads_peer_store", "pa_gather_heads_wait",
    "pa_attention_workspace_bytes", "pa_paged_attention_decode", "pa_paged_attention_varlen",
    "pa_paged_attention_decode_static", "pa_cpu_cache_create", "pa_cpu_cache_free",
    "pa_cpu_cache_is_swapped", "pa_cpu_cache_is_swapped_layer", "pa_cpu_cache_num_swapped", "pa_cpu_cache_block_ptrs", "pa_swap_out",
    "pa_swap_in", "pa_swap_block_bytes",
    "pa_decode_step_host", "pa_kernel_launch_count", "pa_decode_step", "pa_varlen_step_host",
    "pa_cache_check_errors_fast", "pa_paged_attention_decode_rows", "pa_decode_step_rows",
]


class PagedAttnConfig(C.Structure):
    """Same six u32 fields as crates/mlx-sys/src/lib.rs:690-705."""
    _fields_ = [("block_size", C.c_uint32), ("num_blocks", C.c_uint32), ("head_size", C.c_uint32),
                ("num_kv_heads", C.c_uint32), ("num_layers", C.c_uint32), ("dtype", C.c_uint32)]


class PagedAttnError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


_lib = None


def load_library() -> C.CDLL:
    """Load the shared library or raise; never substitutes another implementation."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is not built (run `make -C {os.path.dirname(LIB_PATH)}`); "
            "there is no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, u32, f32, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_float, C.c_size_t
    lib.pa_last_error_string.restype = C.c_char_p
    lib.pa_version.restype = i32
    lib.pa_kernel_launch_count.restype = C.c_uint64
    lib.pa_set_device.argtypes = [i32]
    lib.pa_set_stream.argtypes = [vp]
    lib.pa_cache_create.argtypes = [C.POINTER(PagedAttnConfig), i32, C.POINTER(vp)]
    lib.pa_cache_wrap.argtypes = [C.POINTER(PagedAttnConfig), i32, C.POINTER(vp), C.POINTER(vp),
                                  C.POINTER(vp)]
    lib.pa_cache_create_fp8.argtypes = lib.pa_cache_create.argtypes
    lib.pa_cache_wrap_fp8.argtypes = lib.pa_cache_wrap.argtypes
    lib.pa_cache_is_fp8.argtypes = [vp]
    lib.pa_cache_set_kv_scales.argtypes = [vp, u32, f32, f32]
    lib.pa_cache_get_kv_scales.argtypes = [vp, u32, C.POINTER(f32), C.POINTER(f32)]
    lib.pa_cache_fp8_set_exact_decode.argtypes = [vp, i32]
    lib.pa_gather_heads_peer_store.argtypes = [vp, vp, i64, i32, i32, i32, C.POINTER(vp), C.POINTER(vp),
                                               u32, i32, vp]
    lib.pa_gather_heads_wait.argtypes = [vp, vp, i32, u32, vp]
    lib.pa_cache_free.argtypes = [vp]
    lib.pa_cache_key_ptr.argtypes = [vp, u32]
    lib.pa_cache_key_ptr.restype = vp
    lib.pa_cache_value_ptr.argtypes = [vp, u32]
    lib.pa_cache_value_ptr.restype = vp
    lib.pa_cache_get_config.argtypes = [vp, C.POINTER(PagedAttnConfig)]
    lib.pa_cache_check_errors.argtypes = [vp, vp]
    lib.pa_cache_check_errors_fast.argtypes = [vp, vp]
    lib.pa_paged_attention_decode_rows.argtypes = [vp, u32, vp, vp, vp, vp, vp, i32, i32, i32, i64, i64,
                                                   f32, f32, vp, sz, vp]
    lib.pa_decode_step_rows.argtypes = [vp, u32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i64,
                                        i64, i64, f32, f32, vp, sz, vp]
    lib.pa_reshape_and_cache.argtypes = [vp, u32, vp, vp, vp, i64, i64, i64, vp]
    lib.pa_copy_blocks.argtypes = [vp, u32, vp, i64, vp]
    lib.pa_attention_workspace_bytes.argtypes = [vp]
    lib.pa_attention_workspace_bytes.restype = sz
    lib.pa_paged_attention_decode.argtypes = [vp, u32, vp, vp, vp, vp, i32, i32, i32, i64, i64,
                                              f32, f32, vp, sz, vp]
    lib.pa_paged_attention_decode_static.argtypes = [vp, u32, vp, vp, vp, vp, i32, i32, i32, i64,
                                                     i64, f32, f32, vp]
    lib.pa_paged_attention_varlen.argtypes = [vp, u32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i64,
                                              f32, f32, i32, vp, sz, vp]
    lib.pa_cpu_cache_create.argtypes = [vp]
    lib.pa_cpu_cache_create.restype = vp
    lib.pa_cpu_cache_free.argtypes = [vp]
    lib.pa_cpu_cache_free.restype = None
    lib.pa_cpu_cache_is_swapped.argtypes = [vp, u32]
    lib.pa_cpu_cache_num_swapped.argtypes = [vp]
    lib.pa_cpu_cache_num_swapped.restype = sz
    lib.pa_cpu_cache_is_swapped_layer.argtypes = [vp, u32, u32]
    lib.pa_cpu_cache_block_ptrs.argtypes = [vp, u32, u32, C.POINTER(vp), C.POINTER(vp)]
    lib.pa_swap_out.argtypes = [vp, u32, C.POINTER(u32), sz, vp, vp]
    lib.pa_swap_in.argtypes = [vp, u32, C.POINTER(u32), sz, vp, vp]
    lib.pa_swap_block_bytes.argtypes = [u32, u32, u32, i32, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    lib.pa_swap_block_bytes.restype = None
    lib.pa_qk_norm_rope_and_cache.argtypes = [vp, u32, vp, vp, vp, vp, vp, vp, f32, vp, f32, u32, vp,
                                              i64, i32, i64, i64, i64, i64, vp]
    lib.pa_decode_step_host.argtypes = [vp, u32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, f32]
    lib.pa_varlen_step_host.argtypes = [vp, u32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, f32]
    lib.pa_decode_step.argtypes = [vp, u32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i64,
                                   i64, f32, f32, vp, sz, vp]
    # tier 1
    lib.mlx_paged_attn_create_cache.argtypes = [C.POINTER(PagedAttnConfig)]
    lib.mlx_paged_attn_create_cache.restype = vp
    lib.mlx_paged_attn_free_cache.argtypes = [vp]
    lib.mlx_paged_attn_free_cache.restype = None
    for name in ("mlx_paged_attn_get_key_cache", "mlx_paged_attn_get_value_cache"):
        getattr(lib, name).argtypes = [vp, u32]
        getattr(lib, name).restype = vp
    lib.mlx_paged_attn_reshape_and_cache.argtypes = [vp, u32, vp, vp, vp]
    lib.mlx_paged_attn_reshape_and_cache.restype = None
    lib.mlx_paged_attn_forward.argtypes = [vp, vp, vp, vp, vp, f32, u32, u32]
    lib.mlx_paged_attn_forward.restype = vp
    lib.mlx_paged_attn_copy_blocks.argtypes = [vp, u32, vp]
    lib.mlx_paged_attn_copy_blocks.restype = None
    lib.pa_array_from_device.argtypes = [vp, i32, C.POINTER(i64), sz]
    lib.pa_array_from_device.restype = vp
    lib.pa_array_from_host.argtypes = [vp, i32, C.POINTER(i64), sz]
    lib.pa_array_from_host.restype = vp
    lib.pa_array_data.argtypes = [vp]
    lib.pa_array_data.restype = vp
    lib.mlx_array_ndim.argtypes = [vp]
    lib.mlx_array_ndim.restype = sz
    lib.mlx_array_shape.argtypes = [vp, C.POINTER(i64)]
    lib.mlx_array_shape.restype = None
    lib.mlx_array_dtype.argtypes = [vp]
    lib.mlx_array_dtype.restype = i32
    lib.mlx_array_delete.argtypes = [vp]
    lib.mlx_array_delete.restype = None
    _lib = lib
    return lib


def last_error() -> str:
    return load_library().pa_last_error_string().decode()


def _check(status: int) -> None:
    if status != PA_OK:
        raise PagedAttnError(status, last_error())


def _ptr(x) -> int:
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):  # numpy array (host memory)
        return x.ctypes.data
    raise TypeError(f"cannot take the address of {type(x)}")


def kernel_launch_count() -> int:
    return int(load_library().pa_kernel_launch_count())


class PagedCache:
    """Owner of a PagedAttnCache handle.

    Mirrors the FFI wrapper in crates/mlx-core/src/transformer/paged_attention.rs:53-248
    (new / update_cache / forward / copy_blocks / Drop) on raw device pointers.
    """

    def __init__(self, block_size: int, num_blocks: int, head_size: int, num_kv_heads: int,
                 num_layers: int = 1, dtype: int = 1, device: int = 0, key_pools=None,
                 value_pools=None, fp8: bool = False):
        self.lib = load_library()
        self.cfg = PagedAttnConfig(block_size, num_blocks, head_size, num_kv_heads, num_layers, dtype)
        self.device = device
        self.handle = C.c_void_p()
        self._keep = (key_pools, value_pools)
        self.fp8 = fp8
        create = self.lib.pa_cache_create_fp8 if fp8 else self.lib.pa_cache_create
        wrap = self.lib.pa_cache_wrap_fp8 if fp8 else self.lib.pa_cache_wrap
        if key_pools is None:
            _check(create(C.byref(self.cfg), device, C.byref(self.handle)))
        else:
            kp = (C.c_void_p * num_layers)(*[_ptr(t) for t in key_pools])
            vp = (C.c_void_p * num_layers)(*[_ptr(t) for t in value_pools])
            _check(wrap(C.byref(self.cfg), device, kp, vp, C.byref(self.handle)))
        self._ws = None

    def set_kv_scales(self, k_scale: float, v_scale: float, layer: int = 0) -> None:
        _check(self.lib.pa_cache_set_kv_scales(self.handle, layer, k_scale, v_scale))

    def gather_heads_peer_store(self, local_out, num_tokens: int, heads_local: int, world: int,
                                rank: int, peer_out_ptrs, peer_flag_ptrs, epoch: int,
                                wait: bool = True, stream: int = 0) -> None:
        """Stores this rank's heads into every rank's full-width buffer and (wait=True) waits
        for the others (peer pointers as integers)."""
        outs = (C.c_void_p * world)(*[int(x) for x in peer_out_ptrs])
        flags = (C.c_void_p * world)(*[int(x) for x in peer_flag_ptrs])
        _check(self.lib.pa_gather_heads_peer_store(self.handle, _ptr(local_out), num_tokens,
                                                   heads_local, world, rank, outs, flags, epoch,
                                                   int(wait), stream))

    def gather_heads_wait(self, my_flags, world: int, epoch: int, stream: int = 0) -> None:
        _check(self.lib.pa_gather_heads_wait(self.handle, _ptr(my_flags), world, epoch, stream))

    def fp8_set_exact_decode(self, on: bool) -> None:
        _check(self.lib.pa_cache_fp8_set_exact_decode(self.handle, int(on)))

    def kv_scales(self, layer: int = 0):
        k, v = C.c_float(), C.c_float()
        _check(self.lib.pa_cache_get_kv_scales(self.handle, layer, C.byref(k), C.byref(v)))
        return k.value, v.value

    def close(self) -> None:
        if self.handle:
            self.lib.pa_cache_free(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def key_ptr(self, layer: int = 0) -> int:
        return self.lib.pa_cache_key_ptr(self.handle, layer)

    def value_ptr(self, layer: int = 0) -> int:
        return self.lib.pa_cache_value_ptr(self.handle, layer)

    def workspace_bytes(self) -> int:
        return int(self.lib.pa_attention_workspace_bytes(self.handle))

    def check_errors(self, stream: int = 0) -> None:
        _check(self.lib.pa_cache_check_errors(self.handle, stream))

    def reshape_and_cache(self, key, value, slot_mapping, num_tokens: int, key_stride: int,
                          value_stride: int, layer: int = 0, stream: int = 0) -> None:
        _check(self.lib.pa_reshape_and_cache(self.handle, layer, _ptr(key), _ptr(value),
                                             _ptr(slot_mapping), num_tokens, key_stride,
                                             value_stride, stream))

    def qk_norm_rope_and_cache(self, q_out, q, k, v, q_norm_weight, k_norm_weight, eps: float,
                               positions, rope_base: float, rope_dims: int, slot_mapping,
                               num_tokens: int, num_q_heads: int, q_stride: int, q_out_stride: int,
                               k_stride: int, v_stride: int, layer: int = 0, stream: int = 0) -> None:
        """QK norm + rotary embedding + KV write in one launch (weights may be None)."""
        _check(self.lib.pa_qk_norm_rope_and_cache(
            self.handle, layer, _ptr(q_out), _ptr(q), _ptr(k), _ptr(v),
            _ptr(q_norm_weight) if q_norm_weight is not None else None,
            _ptr(k_norm_weight) if k_norm_weight is not None else None, eps, _ptr(positions),
            rope_base, rope_dims, _ptr(slot_mapping), num_tokens, num_q_heads, q_stride,
            q_out_stride, k_stride, v_stride, stream))

    def copy_blocks(self, block_mapping, num_pairs: int, layer: int = 0, stream: int = 0) -> None:
        _check(self.lib.pa_copy_blocks(self.handle, layer, _ptr(block_mapping), num_pairs, stream))

    def decode(self, out, q, block_tables, context_lens, num_seqs: int, num_q_heads: int,
               max_blocks_per_seq: int, scale: float, workspace, workspace_bytes: int,
               softcap: float = 1.0, q_stride: int | None = None, out_stride: int | None = None,
               layer: int = 0, stream: int = 0) -> None:
        row = num_q_heads * self.cfg.head_size
        _check(self.lib.pa_paged_attention_decode(
            self.handle, layer, _ptr(out), _ptr(q), _ptr(block_tables), _ptr(context_lens),
            num_seqs, num_q_heads, max_blocks_per_seq, q_stride or row, out_stride or row, scale,
            softcap, _ptr(workspace), workspace_bytes, stream))

    def decode_step(self, out, q, key, value, slot_mapping, block_tables, context_lens,
                    num_seqs: int, num_q_heads: int, max_blocks_per_seq: int, scale: float,
                    workspace, workspace_bytes: int, softcap: float = 1.0, layer: int = 0,
                    stream: int = 0) -> None:
        """KV write of the step's tokens + decode attention in one launch."""
        row = num_q_heads * self.cfg.head_size
        kv_row = self.cfg.num_kv_heads * self.cfg.head_size
        _check(self.lib.pa_decode_step(
            self.handle, layer, _ptr(out), _ptr(q), _ptr(key), _ptr(value), _ptr(slot_mapping),
            _ptr(block_tables), _ptr(context_lens), num_seqs, num_q_heads, max_blocks_per_seq,
            row, row, kv_row, kv_row, scale, softcap, _ptr(workspace), workspace_bytes, stream))

    def decode_static(self, out, q, block_tables, context_lens, num_seqs: int, num_q_heads: int,
                      max_blocks_per_seq: int, scale: float, softcap: float = 1.0,
                      q_stride: int | None = None, out_stride: int | None = None, layer: int = 0,
                      stream: int = 0) -> None:
        """Decode attention with the library-resident scratch (no workspace, no allocation)."""
        row = num_q_heads * self.cfg.head_size
        _check(self.lib.pa_paged_attention_decode_static(
            self.handle, layer, _ptr(out), _ptr(q), _ptr(block_tables), _ptr(context_lens),
            num_seqs, num_q_heads, max_blocks_per_seq, q_stride or row, out_stride or row, scale,
            softcap, stream))

    def varlen(self, out, q, block_tables, context_lens, cu_q_lens_host, num_seqs: int,
               num_q_heads: int, max_blocks_per_seq: int, scale: float, workspace,
               workspace_bytes: int, softcap: float = 1.0, max_context_len: int = 0,
               q_stride: int | None = None, out_stride: int | None = None, layer: int = 0,
               stream: int = 0, context_lens_host=None) -> None:
        row = num_q_heads * self.cfg.head_size
        _check(self.lib.pa_paged_attention_varlen(
            self.handle, layer, _ptr(out), _ptr(q), _ptr(block_tables), _ptr(context_lens),
            _ptr(cu_q_lens_host), _ptr(context_lens_host), num_seqs, num_q_heads, max_blocks_per_seq, q_stride or row,
            out_stride or row, scale, softcap, max_context_len, _ptr(workspace), workspace_bytes,
            stream))

    # -- swapping (PagedKVCache::create_cpu_cache / swap_out / swap_in) ----------------
    def create_cpu_cache(self) -> "CpuBlockCache":
        return CpuBlockCache(self)

    def swap_out(self, block_ids, cpu: "CpuBlockCache", layer: int = 0, stream: int = 0) -> None:
        ids = (C.c_uint32 * max(len(block_ids), 1))(*block_ids)
        _check(self.lib.pa_swap_out(self.handle, layer, ids, len(block_ids), cpu.handle, stream))

    def swap_in(self, block_ids, cpu: "CpuBlockCache", layer: int = 0, stream: int = 0) -> None:
        ids = (C.c_uint32 * max(len(block_ids), 1))(*block_ids)
        _check(self.lib.pa_swap_in(self.handle, layer, ids, len(block_ids), cpu.handle, stream))

    def decode_step_host(self, out_host, q_host, k_host, v_host, slots_host, tables_host,
                         lens_host, num_seqs: int, num_q_heads: int, max_blocks_per_seq: int,
                         scale: float, softcap: float = 1.0, layer: int = 0) -> None:
        _check(self.lib.pa_decode_step_host(
            self.handle, layer, _ptr(out_host), _ptr(q_host), _ptr(k_host), _ptr(v_host),
            _ptr(slots_host), _ptr(tables_host), _ptr(lens_host), num_seqs, num_q_heads,
            max_blocks_per_seq, scale, softcap))


    def varlen_step_host(self, out_host, q_host, k_host, v_host, slots_host, tables_host,
                         lens_host, cu_q_lens_host, num_seqs: int, num_q_heads: int,
                         max_blocks_per_seq: int, scale: float, softcap: float = 1.0,
                         layer: int = 0) -> None:
        _check(self.lib.pa_varlen_step_host(
            self.handle, layer, _ptr(out_host), _ptr(q_host), _ptr(k_host), _ptr(v_host),
            _ptr(slots_host), _ptr(tables_host), _ptr(lens_host), _ptr(cu_q_lens_host), num_seqs,
            num_q_heads, max_blocks_per_seq, scale, softcap))


class CpuBlockCache:
    """CpuBlockCache of crates/mlx-paged-attn/src/metal/swap_blocks.rs:15-52."""

    def __init__(self, cache: PagedCache):
        self.lib = cache.lib
        self.handle = self.lib.pa_cpu_cache_create(cache.handle)
        if not self.handle:
            raise PagedAttnError(1, last_error())

    def __del__(self):
        try:
            self.lib.pa_cpu_cache_free(self.handle)
        except Exception:
            pass

    def is_swapped(self, block_id: int, layer: int | None = None) -> bool:
        if layer is not None:
            return bool(self.lib.pa_cpu_cache_is_swapped_layer(self.handle, layer, block_id))
        return bool(self.lib.pa_cpu_cache_is_swapped(self.handle, block_id))

    def num_swapped(self) -> int:
        return int(self.lib.pa_cpu_cache_num_swapped(self.handle))

    def block_ptrs(self, block_id: int, layer: int = 0):
        k, v = C.c_void_p(), C.c_void_p()
        _check(self.lib.pa_cpu_cache_block_ptrs(self.handle, layer, block_id, C.byref(k), C.byref(v)))
        return k.value, v.value
