"""The Rust shim (rust/src/cuda_mm.rs, uncompiled: no Rust toolchain here) must declare every entry point of
include/xn_mm.h with the same argument count -- the check a compiler would not make across the FFI boundary."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header():
    h = open(os.path.join(ROOT, "include", "xn_mm.h")).read()
    h = re.sub(r"/\*.*?\*/", "", h, flags=re.S)
    out = {}
    for name, args in re.findall(r"\b(xn_mm_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", h):
        args = " ".join(args.split())
        out[name] = 0 if args in ("void", "") else args.count(",") + 1
    return out


def _rust():
    r = open(os.path.join(ROOT, "rust", "src", "cuda_mm.rs")).read()
    block = r[r.index('extern "C" {'):]
    block = block[:block.index("\n}\n")]
    out = {}
    for name, args in re.findall(r"pub fn (xn_mm_[a-z0-9_]+)\s*\(([^;]*?)\)\s*(?:->[^;]*)?;", block, flags=re.S):
        args = " ".join(args.split())
        out[name] = 0 if args == "" else args.count(":")
    return out


def test_rust_extern_block_matches_the_header():
    h, r = _header(), _rust()
    assert len(h) >= 40
    assert set(h) == set(r), (sorted(set(h) - set(r)), sorted(set(r) - set(h)))
    assert {k: v for k, v in h.items() if r[k] != v} == {}


def test_build_rs_names_the_source_tree_that_exists():
    b = open(os.path.join(ROOT, "rust", "build.rs")).read()
    assert "xn_b200/csrc" in b and "compute_100a" in b and "rustc-link-lib=dylib=xn_mm" in b
    assert os.path.isdir(os.path.join(ROOT, "xn_b200", "csrc"))
