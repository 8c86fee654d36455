"""The C ABI library loads without a GPU, exports every symbol the header declares, the
host-only transcript entry points match the oracle, and compute entry points fail loudly
(no CPU fallback) when there is no device."""
import ctypes
import os
import random
import re

import pytest

import pyoracle as o

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "zkb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(zk_[a-z0-9_]+)\s*\(", text)) - {"zk_fs_round_fn"})


def test_library_exports_every_declared_symbol():
    from zkes_b200 import _lib
    syms = declared_symbols()
    assert len(syms) >= 20
    for name in syms:
        assert hasattr(_lib.lib, name), f"{name} declared in include/zkb200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"


def test_rust_declarations_cover_the_header():
    """INTEGRATION.md shows the Rust `extern "C"` block a maintainer adds: it must name exactly the functions the
    header declares, each once."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```rust(.*?)```", text, flags=re.S)
    ext = [b for b in blocks if 'extern "C" {' in b]
    assert len(ext) == 1
    names = re.findall(r"pub fn (zk_[a-z0-9_]+)\(", ext[0])
    assert sorted(names) == declared_symbols()
    assert len(names) == len(set(names))


def test_transcript_matches_oracle():
    from zkes_b200 import Transcript
    rnd = random.Random(3)
    a, b = Transcript(b"sumcheck"), o.Transcript(b"sumcheck")
    for i in range(150):
        op = rnd.randrange(4)
        if op == 0:
            m = bytes(rnd.randrange(256) for _ in range(rnd.randrange(0, 400)))
            a.append_message(b"lbl", m)
            b.append_message(b"lbl", m)
        elif op == 1:
            v = rnd.randrange(1 << 64)
            a.append_u64(b"num_var", v)
            b.append_u64(b"num_var", v)
        elif op == 2:
            s = rnd.randrange(o.R_MOD)
            a.append_scalar(b"round_message", s)
            b.append_scalar(b"round_message", s)
        else:
            assert a.challenge_scalar(b"challenge") == b.challenge_scalar(b"challenge")
    a2, b2 = a.clone(), b.clone()
    assert a2.challenge_bytes(b"x", 300) == b2.challenge_bytes(b"x", 300)
    assert a.challenge_bytes(b"x", 300) == b.challenge_bytes(b"x", 300)


def test_no_cpu_fallback_without_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from zkes_b200 import Context
    from zkes_b200._lib import ZkError
    with pytest.raises(ZkError):
        Context(0)


def test_argument_errors_need_no_device():
    from zkes_b200._lib import ZK_ERR_ARG, lib
    assert lib.zk_fold_lsb(None, 3, None, 0, 1, None, None, 0) == ZK_ERR_ARG
    assert lib.zk_sumcheck_linear_prove(None, 2, 2, None, 0, None, None, None, None, None, None, None) == ZK_ERR_ARG
    assert lib.zk_fold_lsb_static(20, ctypes.c_void_p(16), 1, ctypes.c_void_p(16), ctypes.c_void_p(16), None) == ZK_ERR_ARG
