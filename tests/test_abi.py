"""CPU tests of the boundary: the shared library loads, exports every symbol that
include/moe_b200.h declares, rejects bad arguments on the host, and refuses to compute
without a CUDA device (there is no CPU fallback)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "moe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moe_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib_built):
    lib = C.CDLL(str(lib_built))
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in moe_b200.h but not exported"


def test_binding_lists_every_declared_symbol(lib_built):
    from mixtureofexperts_b200 import _lib

    assert sorted(_lib.EXPORTS) == declared_symbols()


def test_binding_return_types_follow_the_header(lib_built):
    """Every export's ctypes restype must be the header's return type: an int64_t truncated to int
    loses the size of weight images of 2 GiB and more; a char* read as int is garbage."""
    from mixtureofexperts_b200 import _lib

    text = open(os.path.join(ROOT, "include", "moe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    decl = dict((name, ret.strip()) for ret, name in re.findall(r"^\s*((?:const\s+)?[a-z0-9_]+\s*\*?)\s*(moe_[a-z0-9_]+)\s*\(", text, flags=re.M))
    assert sorted(decl) == declared_symbols()
    want = {"int": C.c_int, "int64_t": C.c_int64, "const char*": C.c_char_p, "const char *": C.c_char_p}
    for name, ret in decl.items():
        assert getattr(_lib.lib, name).restype is want[ret], (name, ret, getattr(_lib.lib, name).restype)
    assert _lib.lib.moe_layer_weights_image_bytes.restype is C.c_int64


def test_config_struct_matches_header(lib_built):
    from mixtureofexperts_b200 import _lib

    assert C.sizeof(_lib.MoeConfig) == 17 * 4
    assert C.sizeof(_lib.ForwardOutputs) == 7 * C.sizeof(C.c_void_p)


def test_invalid_configs_are_rejected_on_the_host(lib_built):
    from mixtureofexperts_b200 import _lib

    def create(**kw):
        base = dict(num_experts=8, num_shared=0, top_k=2, input_dim=64, hidden_dim=128, output_dim=64,
                    gate_kind=_lib.GATE_TOPK, activation=_lib.ACT_SILU, compute_dtype=_lib.DTYPE_F32,
                    shared_mode=_lib.SHARED_NONE, balance_alpha=0.01, z_loss_weight=0.001, index_base=1,
                    bias_gates_only=0, capacity_factor=1.25, drop_tokens=0, expert_kind=0)
        base.update(kw)
        cfg = _lib.MoeConfig(**base)
        h = C.c_void_p()
        return _lib.lib.moe_layer_create(C.byref(cfg), 0, C.byref(h)), _lib.lib.moe_last_error().decode()

    for kw in (dict(num_experts=0), dict(top_k=9), dict(top_k=0), dict(input_dim=0), dict(activation=9),
               dict(index_base=2), dict(gate_kind=_lib.GATE_SHARED_TOPK), dict(num_shared=1),
               dict(shared_mode=_lib.SHARED_LAYER_BLEND, num_shared=8), dict(drop_tokens=1, capacity_factor=0.0)):
        code, msg = create(**kw)
        assert code == _lib.ERR_INVALID and msg, kw
    code, msg = create(compute_dtype=_lib.DTYPE_BF16, input_dim=60)
    assert code == _lib.ERR_UNSUPPORTED and "multiples of 8" in msg
    code, msg = create(num_experts=200, top_k=2)
    assert code == _lib.ERR_UNSUPPORTED


def test_no_device_means_loud_failure_not_fallback(lib_built):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    import mixtureofexperts_b200 as m

    with pytest.raises(m.MoEError) as ei:
        m.MoELayer(m.create_moe_config(expert_type="gated", activation=m.silu, input_dim=64, hidden_dim=128,
                                       output_dim=64))
    assert ei.value.code == -2 and "no CPU path" in str(ei.value)


def test_null_handles_are_rejected(lib_built):
    from mixtureofexperts_b200 import _lib

    assert _lib.lib.moe_layer_forward(None, None, 0, 1, 0, None, None, None) == _lib.ERR_INVALID
    assert _lib.lib.moe_layer_forward_host(None, None, 0, 1, 0, None, None) == _lib.ERR_INVALID
    assert _lib.lib.moe_layer_destroy(None) == _lib.OK
    assert _lib.lib.moe_compute_gates(_lib.GATE_TOPK, 8, 0, 9, 1, None, 4, None, None, None, None) == _lib.ERR_INVALID


def test_product_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "mixtureofexperts_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "ep.h" or "the oracle for this path" in text.lower(), f


def test_header_compiles_as_c_and_a_c_caller_links(lib_built, tmp_path):
    """The boundary is a C ABI: the header must be plain C99, and a C program linked against the
    library must be able to call it (host-only calls here: version, a rejected config, error text)."""
    import shutil
    import subprocess

    from mixtureofexperts_b200 import _lib

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("gcc not available")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    inc = os.path.join(root, "include")
    src = tmp_path / "caller.c"
    src.write_text(r'''
#include <stdio.h>
#include <string.h>
#include "moe_b200.h"
int main(void) {
    moe_config_t cfg;
    moe_layer_t* h = 0;
    memset(&cfg, 0, sizeof cfg);
    cfg.num_experts = 4; cfg.top_k = 9;            /* top_k > num_experts: refused on the host */
    cfg.input_dim = 8; cfg.hidden_dim = 8; cfg.output_dim = 8;
    int rc = moe_layer_create(&cfg, 0, &h);
    printf("%s|%d|%d|%s\n", moe_version(), (int)sizeof(moe_config_t), rc, moe_last_error());
    return (rc == MOE_ERR_INVALID && h == 0) ? 0 : 1;
}
''')
    exe = tmp_path / "caller"
    lib_dir = os.path.dirname(_lib.LIB_PATH)
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", inc, str(src), "-o", str(exe),
                    "-L", lib_dir, "-lmoe_b200", f"-Wl,-rpath,{lib_dir}"], check=True, capture_output=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    version, size, rc, msg = r.stdout.strip().split("|", 3)
    assert version == _lib.version() and int(size) == C.sizeof(_lib.MoeConfig) and "top_k" in msg
