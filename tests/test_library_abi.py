"""CPU-only checks of the C-ABI boundary: the library builds and loads without a GPU, exports
every symbol the header declares, and the ctypes structures match the C layout."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

from conftest import ROOT
from qutai_b200 import lib
from qutai_b200.storage import bf16_bits

HEADER = os.path.join(ROOT, "include", "qutai_moe.h")


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    return sorted(set(re.findall(r"\b(qmoe_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_binding_binds():
    names = declared_functions()
    assert len(names) >= 35
    assert sorted(lib.SIGNATURES) == names


def test_library_loads_and_exports_every_declared_symbol(library_path):
    handle = ctypes.CDLL(library_path)
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} is declared in include/qutai_moe.h but not exported"
    loaded = lib.load()
    assert loaded.qmoe_version() == 100
    assert loaded.qmoe_timing_classes() >= 10


def test_size_helpers_need_no_device(library_path):
    assert lib.rows_bound(16384, 8, 2) == 33792            # 32768 + 8 * 127, rounded up to 128
    assert lib.rows_bound(1, 1, 1) == 128
    assert lib.rows_bound(64, 64, 6) % lib.ROW_PAD == 0 and lib.rows_bound(64, 64, 6) >= 384 + 64 * 127
    assert lib.route_blocks(1) == 1 and lib.route_blocks(32) == 1 and lib.route_blocks(33) == 2
    scratch = int(lib.load().qmoe_router_scratch_bytes(4096, 8, 1024))
    assert scratch >= 4096 * 6 * 32 * 2 + 9 * 32 * 1024 * 2      # split gradients + split weights at least
    assert int(lib.load().qmoe_router_grad_partials(4096, 8, 1024)) * 4 >= scratch


def test_ctypes_structures_match_the_c_layout(tmp_path):
    source = tmp_path / "layout.c"
    fields = {"qmoe_route_t": [f[0] for f in lib.Route._fields_],
              "qmoe_experts_t": [f[0] for f in lib.Experts._fields_],
              "qmoe_layer_t": [f[0] for f in lib.Layer._fields_],
              "qmoe_block_t": [f[0] for f in lib.Block._fields_],
              "qmoe_head_t": [f[0] for f in lib.Head._fields_],
              "qmoe_attention_t": [f[0] for f in lib.Attention._fields_],
              "qmoe_optim_item_t": [f[0] for f in lib.OptimItem._fields_]}
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void) {"]
    for struct, names in fields.items():
        lines.append(f'printf("{struct} %zu\\n", sizeof({struct}));')
        for name in names:
            lines.append(f'printf("{struct}.{name} %zu\\n", offsetof({struct}, {name}));')
    lines += ["return 0; }"]
    source.write_text("\n".join(lines))
    binary = tmp_path / "layout"
    subprocess.run(["gcc", "-o", str(binary), str(source)], check=True)
    reported = dict(line.rsplit(" ", 1) for line in subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout.splitlines())
    for struct, cls in (("qmoe_route_t", lib.Route), ("qmoe_experts_t", lib.Experts), ("qmoe_layer_t", lib.Layer),
                        ("qmoe_block_t", lib.Block), ("qmoe_head_t", lib.Head), ("qmoe_attention_t", lib.Attention),
                        ("qmoe_optim_item_t", lib.OptimItem)):
        assert int(reported[struct]) == ctypes.sizeof(cls)
        for name, _ in cls._fields_:
            assert int(reported[f"{struct}.{name}"]) == getattr(cls, name).offset, (struct, name)


def test_argument_errors_raise_value_error_without_a_device(library_path):
    with pytest.raises(ValueError):
        lib.call("qmoe_route", None, 0, 0)
    assert "null" in lib.last_error()
    route = lib.Route()
    route.tokens, route.experts, route.top_k = 4, 300, 2
    with pytest.raises(ValueError):
        lib.call("qmoe_route", ctypes.byref(route), 1, 0)
    with pytest.raises(ValueError):
        lib.call("qmoe_cast_bf16", 8, 16, 4, 0)  # misaligned addresses
    head = lib.Head()
    head.batch, head.time, head.width, head.vocab, head.rows_bound = 2, 1, 8, 16, 128
    with pytest.raises(ValueError):
        lib.call("qmoe_head_forward", ctypes.byref(head), 0)   # a sequence of one position has no target
    head.time, head.rows_bound = 3, 100
    with pytest.raises(ValueError):
        lib.call("qmoe_head_forward", ctypes.byref(head), 0)   # rows_bound is not a multiple of 128


def test_bf16_rounding_on_the_host():
    assert bf16_bits(1.0) == 0x3F80
    assert bf16_bits(1.0 + 2 ** -8) == 0x3F80          # tie -> even
    assert bf16_bits(1.0 + 3 * 2 ** -8) == 0x3F82      # tie -> even (up)
    assert bf16_bits(-2.5) == 0xC020


def test_product_does_not_import_the_oracle():
    package = os.path.join(ROOT, "qutai_b200")
    for folder, _, files in os.walk(package):
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(folder, name), encoding="utf-8").read()
                assert "oracle" not in text.replace("the oracle", ""), f"{name} refers to oracle/"
