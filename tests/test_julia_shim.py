"""julia/B200Device.jl cannot be run where this library is built (no Julia): what can be checked is that every
ccall in it names an entry point the header declares and passes as many arguments as the declaration has, with
integer / float / pointer kinds that agree."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_decls():
    text = open(os.path.join(ROOT, "include", "luminal_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(?:int32_t|const char\*)\s+(lmb200_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        params = [p.strip() for p in m.group(2).split(",") if p.strip() and p.strip() != "void"]
        out[m.group(1)] = params
    return out


def kind_c(p):
    if "*" in p or "[" in p:
        return "ptr"
    if p.startswith("float"):
        return "f32"
    if re.match(r"(u?int64_t|lmb200_ctx|lmb200_model|lmb200_session|lmb200_whisper_encoder)\b", p):
        return "i64"
    return "i32"


def kind_jl(t):
    t = t.strip()
    if t.startswith(("Ptr{", "Ref{")) or t == "Cstring":
        return "ptr"
    return {"Float32": "f32", "Int64": "i64", "UInt64": "i64", "Int32": "i32"}[t]


def split_types(s):
    out, depth, cur = [], 0, ""
    for ch in s:
        if ch == "{":
            depth += 1
        if ch == "}":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur)
    return [t for t in (x.strip() for x in out) if t]


def test_every_ccall_matches_a_declaration():
    decls = header_decls()
    src = open(os.path.join(ROOT, "julia", "B200Device.jl")).read()
    calls = []
    for m in re.finditer(r"ccall\(\(:(lmb200_[a-z0-9_]+), LIB\),\s*(\w+),\s*\(", src):
        depth, i = 1, m.end()
        while depth:                                   # the argument-type tuple, parentheses balanced
            depth += {"(": 1, ")": -1}.get(src[i], 0)
            i += 1
        calls.append((m.group(1), m.group(2), src[m.end():i - 1]))
    assert len(calls) >= 40
    for name, ret, types in calls:
        assert name in decls, f"{name} is not declared in the header"
        jl = split_types(types)
        assert len(jl) == len(decls[name]), f"{name}: {len(jl)} ccall argument types, {len(decls[name])} parameters"
        for t, p in zip(jl, decls[name]):
            assert kind_jl(t) == kind_c(p), f"{name}: Julia type {t} against C parameter '{p}'"
        assert ret == ("Cstring" if name == "lmb200_last_error" else "Int32")


def test_every_reference_op_has_a_method():
    src = open(os.path.join(ROOT, "julia", "B200Device.jl")).read()
    ops = ["Add", "Mul", "Mod", "LessThan", "Max", "Log2", "Exp2", "Sin", "Cos", "Sqrt", "Recip", "ReLU", "Contiguous",
           "FusedMulAdd", "FusedAddReLU", "SumReduce", "MaxReduce", "MatMul", "Permute", "Reshape", "Expand", "Slice", "Pad",
           "Unfold", "FlashAttentionOp", "Function"]
    for op in ops:
        assert re.search(rf"Luminal\.execute_op!\(out::B200Array, (?:op)?::Luminal\.{op}\b", src), op
