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


def test_backend_source_calls_only_declared_functions_with_the_declared_arity():
    """bindings/rust/cuda_b200.rs (the `Backend` implementation over the library, uncompiled like the
    declarations): every `rtb_*` call names a declared function and passes as many arguments as it takes,
    and the op codes it carries equal the ctypes binding's."""
    from rtensors_b200 import _lib as L
    src = open(os.path.join(ROOT, "bindings", "rust", "cuda_b200.rs")).read()
    decl = _rust_functions()
    calls = 0
    for m in re.finditer(r"\b(rtb_\w+)\s*\(", src):
        name = m.group(1)
        assert name in decl, name
        depth, i, args, cur = 1, m.end(), [], ""
        while depth:                                   # split the argument list at top-level commas
            ch = src[i]
            if ch in "([{":
                depth += 1
            elif ch in ")]}":
                depth -= 1
                if depth == 0:
                    break
            if ch == "," and depth == 1:
                args.append(cur)
                cur = ""
            else:
                cur += ch
            i += 1
        if cur.strip():
            args.append(cur)
        assert len(args) == decl[name], (name, len(args), decl[name])
        calls += 1
    assert calls >= 25
    for name, value in re.findall(r"pub const (\w+): i32 = (\d+);", src):
        assert getattr(L, name) == int(value), name
    for family in ("neg", "relu", "sigmoid", "silu", "tanh", "abs", "sqrt", "ln", "expm1", "ln1p", "floor", "ceil", "round", "trunc",
                   "sin", "cos", "tan", "asin", "acos", "atan", "sinh", "cosh", "asinh", "acosh", "atanh", "rsqrt", "reciprocal",
                   "square", "cube", "exp", "sign"):
        assert re.search(r"unary_family!\s*\{\s*%s\s*," % family, src), family
    for family in ("add", "sub", "mul", "div", "log", "log1p", "leaky_relu", "elu"):
        assert re.search(r"scalar_family!\s*\{\s*%s\s*," % family, src), family
