"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the
header declares, and rejects bad arguments before touching a device."""
import ctypes as C
import os
import re

import pytest

import paged_attn_b200 as pa

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADERS = [os.path.join(ROOT, "include", n) for n in ("paged_attn_b200.h", "paged_attn_b200_host.h")]


def declared_functions():
    names = []
    for header in HEADERS:
        text = open(header).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b((?:pa|mlx)_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_and_binding_list_the_same_symbols():
    from paged_attn_b200 import host
    assert declared_functions() == sorted(pa.EXPORTED_SYMBOLS + host.HOST_SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = pa.load_library()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} missing from {pa.LIB_PATH}"


def test_no_torch_or_oracle_in_the_library():
    # The shipped library must not depend on the oracle or on a tensor library.
    import subprocess
    out = subprocess.run(["ldd", pa.LIB_PATH], capture_output=True, text=True).stdout
    # library names only: the load addresses ldd prints are random hex and may spell anything
    names = " ".join(line.split("(0x")[0] for line in out.splitlines())
    assert names.strip()
    assert "liboracle" not in names and "torch" not in names and "c10" not in names


def test_version_and_error_string():
    lib = pa.load_library()
    assert lib.pa_version() >= 100
    assert isinstance(pa.last_error(), str)


@pytest.mark.parametrize("field,value,status", [
    ("block_size", 64, 1),      # crates/mlx-paged-attn/src/config.rs:144-160: block 64 rejected
    ("head_size", 100, 1),      # head 100 rejected
    ("num_blocks", 0, 1),
    ("dtype", 7, 1),
    ("dtype", 2, 2),            # f32 accepted by the reference, not built here
])
def test_config_validation_needs_no_device(field, value, status):
    lib = pa.load_library()
    cfg = pa.PagedAttnConfig(16, 8, 128, 2, 1, 1)
    setattr(cfg, field, value)
    handle = C.c_void_p()
    assert lib.pa_cache_create(C.byref(cfg), 0, C.byref(handle)) == status
    assert not handle.value
    assert pa.last_error()
    assert lib.mlx_paged_attn_create_cache(C.byref(cfg)) is None


def test_null_arguments_are_rejected():
    lib = pa.load_library()
    assert lib.pa_cache_create(None, 0, C.byref(C.c_void_p())) == 1
    assert lib.pa_reshape_and_cache(None, 0, None, None, None, 1, 1, 1, None) == 1
    assert lib.pa_paged_attention_decode(None, 0, None, None, None, None, 1, 1, 1, 1, 1, 1.0, 1.0,
                                         None, 0, None) == 1
    assert lib.pa_copy_blocks(None, 0, None, 1, None) == 1
    assert lib.pa_cache_free(None) == 0
    assert lib.pa_attention_workspace_bytes(None) == 0
    assert lib.mlx_paged_attn_forward(None, None, None, None, None, 1.0, 16, 0) is None
    lib.mlx_paged_attn_reshape_and_cache(None, 0, None, None, None)   # silent no-op
    lib.mlx_paged_attn_copy_blocks(None, 0, None)
    lib.mlx_array_delete(None)


def test_compute_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(pa.PagedAttnError):
        pa.PagedCache(16, 8, 128, 2)


def test_swap_block_sizes():
    # crates/mlx-paged-attn/src/metal/swap_blocks.rs:265-312: 16384 B per block for 4 heads x 128 x 16
    # in 16-bit storage, 8192 B with an fp8 cache
    import ctypes as C
    lib = pa.load_library()
    k, v = C.c_uint64(), C.c_uint64()
    lib.pa_swap_block_bytes(4, 128, 16, 0, C.byref(k), C.byref(v))
    assert (k.value, v.value) == (16384, 16384)
    lib.pa_swap_block_bytes(4, 128, 16, 1, C.byref(k), C.byref(v))
    assert (k.value, v.value) == (8192, 8192)


def test_plain_c_program_links_and_runs(tmp_path):
    """The headers are C (not only C++) and the shared object is usable from a C program
    without Python in between; only entry points that need no GPU are called."""
    import shutil
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cc = shutil.which("gcc")
    if cc is None:
        pytest.skip("no C compiler")
    libdir = os.path.join(root, "mlx-node_b200")
    exe = str(tmp_path / "c_abi_host_smoke")
    subprocess.run([cc, "-std=c11", "-Wall", "-Werror", "-I", os.path.join(root, "include"),
                    os.path.join(root, "tests", "c_abi_host_smoke.c"), "-o", exe, "-L", libdir,
                    "-lpaged_attn_b200", f"-Wl,-rpath,{libdir}"], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    words = r.stdout.split()
    assert words[0] == "version" and int(words[1]) >= 100
    assert words[-5:] == ["shard", "4", "8", "16", "32"] and words[words.index("hash") + 1] == "1"
