"""CPU-only checks of the drop-in boundary: the C-ABI library loads, exports exactly the symbols
include/aet_b200.h declares, refuses to run without a GPU (no fallback), and the cfg readers agree."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def header_functions():
    text = open(os.path.join(ROOT, "include", "aet_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aet_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(aet):
    lib = aet.lib()
    declared = header_functions()
    assert len(declared) > 60
    for name in declared:
        assert hasattr(lib, name), "libaet_b200.so does not export " + name
    assert sorted(aet.EXPORTS) == declared, "python binding and header disagree"
    assert b"sm_100a" in lib.aet_version()


def test_no_cpu_fallback(aet):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(aet.AetError) as e:
        aet.Context(0)
    assert "no CPU path" in str(e.value)


def test_null_arguments_return_errors_not_crashes(aet):
    lib = aet.lib()
    assert lib.aet_tensor_write(None, None) == -1
    assert lib.aet_network_update(None) == -1
    assert lib.aet_layer_update(None, 1, 0.1, 0.9, 0.0, 1.0) == -1
    assert lib.aet_network_create_ex(None, b"[net]", 1, 0) is None
    assert b"null" in lib.aet_last_error()


def test_cfg_reader_defaults(aet):
    from oracle import cfgfile
    text = open(os.path.join(aet.CFG_DIR, "cifar_small.cfg")).read()
    net, layers = cfgfile.network_spec(text)
    assert net["batch"] == 128 and (net["c"], net["h"], net["w"]) == (3, 32, 32)
    assert [l["type"] for l in layers] == [0, 1, 0, 1, 0, 1, 0, 2, 3]
    assert layers[0]["pad"] == 1 and layers[6]["pad"] == 0 and layers[6]["activation"] == 0
    assert layers[1]["pad"] == 1            # maxpool default padding = size - 1
    net2, _ = cfgfile.network_spec("[net]\nbatch=64\nsubdivisions=4\nchannels=3\nheight=8\nwidth=8\n")
    assert net2["batch"] == 16              # [net] batch is divided by subdivisions
    _, dl = cfgfile.network_spec("[net]\nchannels=1\nheight=4\nwidth=4\n[convolutional]\nfilters=2\n")
    assert dl[0]["activation"] == 3         # the reference's default activation is logistic (dnn/NetworkFactory.c:103)
    with pytest.raises(KeyError):
        cfgfile.network_spec("[net]\nchannels=1\nheight=4\nwidth=4\n[convolutional]\nfilters=2\nactivation=gelu\n")
    anet, alayers = cfgfile.network_spec(open(os.path.join(aet.CFG_DIR, "alexnet_style.cfg")).read())
    assert sum(1 for l in alayers if l["type"] == 0) == 8 and alayers[1]["pad"] == 0


def test_every_kernel_waits_for_its_predecessor_before_touching_global_memory():
    """Kernels are launched with programmatic stream serialization, so each one must call pdl_enter()
    (griddepcontrol.wait) itself: a kernel without it would race with the tail of the previous launch."""
    import re
    csrc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "aet-cnn_b200", "csrc")
    checked = 0
    for fn in sorted(os.listdir(csrc)):
        if not fn.endswith((".cu", ".cuh")):
            continue
        src = open(os.path.join(csrc, fn)).read()
        for m in re.finditer(r"__global__", src):
            start = src.find("{", src.find(")", m.start()))
            depth, k = 0, start
            while True:
                if src[k] == "{":
                    depth += 1
                elif src[k] == "}":
                    depth -= 1
                    if depth == 0:
                        break
                k += 1
            assert "pdl_enter()" in src[start:k], "%s: kernel at offset %d never calls pdl_enter()" % (fn, m.start())
            checked += 1
    assert checked >= 30
