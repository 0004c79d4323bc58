"""bindings/rust/rt_b200_sys.rs is text (no Rust toolchain in the build image): keep it honest against
the C header and the built library -- same function names, same parameter counts, every name exported."""
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    h = open(os.path.join(ROOT, "include", "rt_b200.h")).read()
    h = re.sub(r"/\*.*?\*/", "", h, flags=re.S)
    h = re.sub(r"//[^\n]*", "", h)
    out = {}
    for name, args in re.findall(r"\b(rtb_\w+)\s*\(([^;{]*?)\)\s*;", h):
        args = args.strip()
        out[name] = 0 if args in ("", "void") else len(re.split(r",", args))
    return out


def _rust_functions():
    r = open(os.path.join(ROOT, "bindings", "rust", "rt_b200_sys.rs")).read()
    out = {}
    for name, args in re.findall(r"pub fn (rtb_\w+)\(([^)]*)\)", r):
        out[name] = 0 if not args.strip() else len(args.split(","))
    return out


def test_rust_declarations_match_the_c_header():
    c, r = _header_functions(), _rust_functions()
    assert len(c) > 60
    assert set(c) == set(r), (sorted(set(c) - set(r)), sorted(set(r) - set(c)))
    for name in c:
        assert c[name] == r[name], (name, c[name], r[name])


def test_every_rust_declaration_is_exported_by_the_library():
    import rtensors_b200 as rt
    rt.lib()
    syms = subprocess.run(["nm", "-D", "--defined-only", os.path.join(ROOT, "rtensors_b200", "librt_b200.so")],
                          capture_output=True, text=True, check=True).stdout
    exported = set(re.findall(r" T (rtb_\w+)", syms))
    missing = sorted(set(_rust_functions()) - exported)
    assert not missing, missing
