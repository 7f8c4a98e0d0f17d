"""The C-ABI boundary without a GPU: the library loads, exports every symbol include/blum.h declares,
its host-side generators agree with the oracle's, and host-only error paths behave."""
import ctypes as C
import os

import numpy as np

from luminal_b200 import _lib, runtime


def test_library_exports_every_declared_symbol():
    protos = _lib.all_declared_functions()        # include/blum.h and include/blum_dev.h
    assert len(protos) >= 70
    raw = C.CDLL(_lib.LIB_PATH)
    missing = [n for n in protos if not hasattr(raw, n)]
    assert not missing, missing
    for must in ("blum_q8_0_matmul", "blum_q8_0_gather", "blum_rmsnorm", "blum_rope_interleaved", "blum_kv_append_paged",
                 "blum_attn_decode_paged", "blum_attn_prefill_paged", "blum_swiglu", "blum_argmax", "blum_llama_decode",
                 "blum_q8_0_weight_from_gguf_bytes"):
        assert must in protos


def test_every_product_declaration_names_its_reference_counterpart():
    """include/blum.h is the drop-in boundary: the comment that precedes a declaration (or the section comment above it)
    cites the reference interface it stands in for (a path in the luminal tree) or says that there is none."""
    import re
    text = open(_lib.HEADER_PATH).read()
    protos = _lib.declared_functions()
    dev = _lib.declared_functions(_lib.DEV_HEADER_PATH)
    assert not set(protos) & set(dev)
    cite = re.compile(r"crates/|src/|examples/|[Nn]o counterpart|absent in the reference|reference has|reference's|luminal (has|hard-codes)")
    uncited = []
    for name in protos:
        at = re.search(r"^(?:const\s+)?[A-Za-z_][\w \*]*\b%s\(" % name, text, flags=re.M).start()      # the declaration, not a mention
        comments = re.findall(r"/\*.*?\*/", text[:at], flags=re.S)
        # the nearest comment, or the nearest section comment (one that opens with a dashed rule)
        nearest = comments[-1] if comments else ""
        section = next((c for c in reversed(comments) if "-----" in c), "")
        if not (cite.search(nearest) or cite.search(section)):
            uncited.append(name)
    assert not uncited, uncited


def test_no_torch_types_in_signatures():
    text = open(_lib.HEADER_PATH).read()
    assert "torch" not in text and "at::" not in text and "std::" not in text
    assert 'extern "C"' in text


def test_version_and_null_context():
    lib = _lib.load()
    assert b"sm_100a" in lib.blum_version()
    assert lib.blum_sync(None) == _lib.ERR_INVALID
    assert lib.blum_q8_0_matmul(None, None, None, 0, None, 0, 1) == _lib.ERR_INVALID
    assert lib.blum_last_error(None) == b"null context"
    assert lib.blum_q8_0_weight_rows(None) == -1
    assert lib.blum_kv_seq_len(None, 0) == -1


def test_generators_identical_in_library_and_oracle(orc):
    for seed, tid in ((0, 1), (1, 7), (3, 2 ** 40 + 5)):
        assert np.array_equal(runtime.gen_q8_quants(seed, tid, 10007), orc.gen_q8_quants(seed, tid, 10007))
        assert np.array_equal(runtime.gen_q8_scales(seed, tid, 5003), orc.gen_q8_scales(seed, tid, 5003))
        assert np.array_equal(runtime.gen_normal(seed, tid, 5003, 0.02), orc.gen_normal(seed, tid, 5003, 0.02))
        assert np.array_equal(runtime.gen_token_ids(seed, tid, 64, 128256), orc.gen_token_ids(seed, tid, 64, 128256))


def test_tensor_ids_are_fnv1a_of_gguf_names():
    from helpers import fnv1a
    lib = _lib.load()
    for name in ("token_embd.weight", "blk.0.attn_q.weight", "blk.31.ffn_down.weight", "output.weight"):
        assert lib.blum_llama_tensor_id(name.encode()) == fnv1a(name)


def test_host_pack_matches_oracle_and_bf16_rounding(orc):
    q = runtime.gen_q8_quants(2, 1, 64 * 128).reshape(64, 128)
    d = runtime.gen_q8_scales(2, 1, 64 * 4).reshape(64, 4)
    assert np.array_equal(runtime.pack_gguf_q8_0(q, d), orc.q8_pack(q, d))
    a = np.concatenate([runtime.gen_normal(2, 2, 4096), np.array([0.0, -0.0, 1e-40, 3.4e38, np.inf], np.float32)])
    assert np.array_equal(runtime.f32_to_bf16_bits(a), orc.bf16_bits(a))
    assert np.array_equal(runtime.round_to_dtype(a, _lib.BF16), orc.round_bf16(a))


def test_attn_scratch_size_formula():
    lib = _lib.load()
    assert lib.blum_attn_decode_scratch_bytes(64, 32, 128, 8) == 64 * 32 * 8 * 130 * 4
    assert lib.blum_attn_decode_scratch_bytes(64, 32, 128, 1) == 0


def test_product_has_no_oracle_dependency():
    """Nothing under luminal_b200/ may import or link the oracle."""
    root = os.path.join(os.path.dirname(_lib.HERE), "luminal_b200")
    for dirpath, _, files in os.walk(root):
        if "_build" in dirpath:
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                for needle in ("import oracle", "from oracle", "liboracle", "oracle/", "oracle."):
                    assert needle not in text, (dirpath, f, needle)


def test_rust_ffi_declarations_follow_the_header():
    """luminal_b200/rust/src/ffi.rs is generated from include/blum.h: it must be the generator's current output, declare
    every entry point of the header with the same number of arguments, and lib.rs may only call what it declares."""
    import importlib.util
    import re
    here = os.path.dirname(os.path.abspath(__file__))
    gen = os.path.join(here, "..", "luminal_b200", "rust", "gen_ffi.py")
    spec = importlib.util.spec_from_file_location("gen_ffi", gen)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    text = open(mod.OUT).read()
    assert text == mod.render(), "ffi.rs is stale: run python luminal_b200/rust/gen_ffi.py"
    protos = _lib.declared_functions()
    for name, (_, argtypes) in protos.items():
        m = re.search(r"pub fn %s\(([^)]*)\)" % name, text)
        assert m, name
        nargs = len([a for a in m.group(1).split(",") if a.strip()])
        assert nargs == len(argtypes), (name, nargs, len(argtypes))
    lib_rs = open(os.path.join(os.path.dirname(mod.OUT), "lib.rs")).read()
    for called in set(re.findall(r"ffi::(blum_[a-z0-9_]+)\(", lib_rs)):
        assert called in protos, called
