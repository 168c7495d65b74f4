"""The Zig module that stands in for tensor_math_standard.zig cannot be compiled here (no Zig toolchain), so it is
checked mechanically: every name of the reference's table that lies on the inference path, and every
`tensMath.<name>` the code generator or the hand-kept generated samples use, must exist in the shim with the
reference's parameter count; every extern declaration must name a function of include/zant_b200.h; and the
status mapping must cover every code of the header's enum.  The reference's side of the comparison is
tests/golden/tensor_math_names.json (written by tests/golden/make_name_table.py from the reference's sources)."""
import json
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "z-ant_b200", "zig", "tensor_math_b200.zig")
HEADER = os.path.join(ROOT, "include", "zant_b200.h")
TABLE = json.load(open(os.path.join(ROOT, "tests", "golden", "tensor_math_names.json")))


def split_params(text):
    out, depth, cur = [], 0, ""
    for ch in text:
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur.strip()); cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur.strip())
    return out


def shim_symbols():
    src = open(SHIM).read()
    fns = {}
    for m in re.finditer(r"^pub fn (\w+)\((.*)\) (!?[\w\[\]\(\)\.]+) \{$", src, flags=re.M):
        fns[m.group(1)] = split_params(m.group(2))
    for m in re.finditer(r"^pub const (\w+) = (\w+);$", src, flags=re.M):
        if m.group(2) in fns:
            fns[m.group(1)] = fns[m.group(2)]
    types = set(re.findall(r"^pub const (\w+) = (?:enum|opaque|error)", src, flags=re.M))
    externs = re.findall(r"^extern fn (\w+)\(", src, flags=re.M)
    return src, fns, types, externs


def test_every_hot_path_name_exists_with_the_reference_parameter_count():
    _src, fns, types, _ = shim_symbols()
    problems = []
    for row in TABLE["names"]:
        if row["scope"] != "hot-path":
            continue
        name = row["name"]
        if row["kind"] == "type" or row["params"] is None:
            if name not in fns and name not in types:
                problems.append(f"{name}: missing ({row['file']})")
            continue
        if name not in fns:
            problems.append(f"{name}: missing (reference: {row['file']}:{row['line']})")
        elif len(fns[name]) != len(row["params"]):
            problems.append(f"{name}: {len(fns[name])} parameters, the reference has {len(row['params'])} ({row['file']}:{row['line']})")
        else:
            # comptime parameters sit at the same positions
            ours = [p.startswith("comptime") for p in fns[name]]
            theirs = [p.startswith("comptime") for p in row["params"]]
            if ours != theirs:
                problems.append(f"{name}: comptime parameters differ ({row['file']}:{row['line']})")
    assert not problems, "\n".join(problems)
    assert sum(r["scope"] == "hot-path" for r in TABLE["names"]) >= 35


def test_every_name_generated_code_uses_resolves():
    _src, fns, types, _ = shim_symbols()
    missing = [f"{e['name']} ({e['first_use']})" for e in TABLE["used_by_generated_code"] if e["name"] not in fns and e["name"] not in types]
    assert not missing, missing


def test_quantized_names_are_present():
    _src, fns, _types, _ = shim_symbols()
    for name in ("qlinearconv_lean", "qlinearmatmul_lean", "quantizelinear_lean", "dequantizelinear_lean"):
        assert name in fns, name


def test_extern_declarations_match_the_header():
    _src, _fns, _types, externs = shim_symbols()
    header = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    declared = {}
    for m in re.finditer(r"\b(zant_b200_\w+)\s*\(([^;]*?)\)\s*;", header, flags=re.S):
        args = m.group(2).strip()
        declared[m.group(1)] = 0 if args in ("", "void") else len(split_params(args))
    src = open(SHIM).read()
    assert len(externs) >= 35
    for name in externs:
        assert name in declared, f"{name} is not declared in include/zant_b200.h"
        sig = re.search(r"^extern fn " + name + r"\((.*)\) \w+;$", src, flags=re.M).group(1)
        assert len(split_params(sig)) == declared[name], f"{name}: argument count differs from the header"


def test_status_mapping_is_total():
    src = open(SHIM).read()
    header = open(HEADER).read()
    enum = header[header.index("typedef enum zant_status"):header.index("} zant_status;")]
    codes = [int(v) for v in re.findall(r"=\s*(-?\d+)", enum)]
    check = src[src.index("fn check(status: i32) !void"):]
    check = check[:check.index("};")]
    arms = {int(v) for v in re.findall(r"^\s*(-?\d+) =>", check, flags=re.M)}
    assert set(codes) <= arms, sorted(set(codes) - arms)
    # each arm names the error the header's comment promises
    for code, zig_name in re.findall(r"^\s*(-\d+) => \w+\.(\w+),", check, flags=re.M):
        c_name = re.search(r"ZANT_E_(\w+) = " + code + r"\b", enum).group(1)
        assert c_name.replace("_", "").lower() == zig_name.lower(), (code, c_name, zig_name)
