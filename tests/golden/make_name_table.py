"""Writes tests/golden/tensor_math_names.json: the name table generated code links against
(src/Core/Tensor/TensorMath/tensor_math_standard.zig in the Z-Ant tree), each `pub const NAME = lib.fn`
resolved to the function it aliases with file:line and parameter list.  Run where the reference checkout
is available:  python tests/golden/make_name_table.py /path/to/Z-Ant
The test that uses the table (tests/test_zig_shim.py) needs only the JSON."""
import json
import os
import re
import sys

# Names that are not on the inference path (training passes, debugging helpers, layout utilities that only the
# reference's own CPU kernels use) and are therefore not provided by the device back end's module.
OUT_OF_SCOPE = {
    "convolution_backward_biases": "training", "convolution_backward_weights": "training", "convolution_backward_input": "training",
    "pool_tensor": "training", "multidim_pooling": "training", "pool_forward": "training", "pool_backward": "training",
    "ReLU_backward": "training", "leakyReLU_backward": "training", "sigmoid_backward": "training", "softmax_backward": "training",
    "multidim_convolution_with_bias": "training-era API", "convolve_tensor_with_bias": "internal step of Conv",
    "calculateStrides": "CPU helper", "transpose2D": "CPU helper", "transposeDefault": "CPU helper", "transposeLastTwo": "CPU helper",
    "addPaddingAndDilation": "CPU helper", "flip": "training", "split": "generator stub (OperationWIP)", "get_split_output_shapes": "generator stub",
    "dot_product_tensor_flat": "not emitted", "mean": "not emitted", "sub_tensors": "generator stub (Sub)", "isOneHot": "debug helper",
    "isSafe": "debug helper", "equal": "debug helper",
    # allocating forms: generated code calls the lean forms; these remain available from the reference's own files
    "reshape": "allocating form", "gather": "allocating form", "unsqueeze": "allocating form", "mat_mul": "allocating form",
    "gemm": "allocating form", "onnx_maxpool": "allocating form", "sum_tensors": "allocating form", "sum_tensor_list": "allocating form",
    "shape_onnx": "allocating form", "slice_onnx": "allocating form", "mul": "allocating form", "div": "allocating form",
    "tanh": "allocating form", "ceil": "allocating form", "reduce_mean": "allocating form", "ReLU": "allocating form",
    "leakyReLU": "allocating form", "sigmoid": "allocating form", "softmax": "allocating form", "transpose_onnx": "allocating form",
}


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
    return [re.sub(r"//.*", "", p).strip() for p in out if re.sub(r"//.*", "", p).strip()]


def find_fn(src_dir, file, fn):
    lines = open(os.path.join(src_dir, file)).read().split("\n")
    for i, line in enumerate(lines):
        m = re.match(r"\s*pub (?:inline )?fn " + re.escape(fn) + r"\s*\(", line)
        if not m:
            continue
        text, depth, j, k = "", 0, i, line.index("(", m.start())
        while True:
            for ch in lines[j][k:]:
                if ch == "(":
                    depth += 1
                    if depth == 1:
                        continue
                elif ch == ")":
                    depth -= 1
                    if depth == 0:
                        return i + 1, split_params(text)
                text += ch
            text += "\n"; j += 1; k = 0
    return None, None


def main(ref):
    d = os.path.join(ref, "src", "Core", "Tensor", "TensorMath")
    table = open(os.path.join(d, "tensor_math_standard.zig")).read().split("\n")
    imports = dict(re.findall(r'const (\w+) = @import\("([\w.]+)"\);', "\n".join(table)))
    rows = []
    for n, line in enumerate(table):
        m = re.match(r"\s*pub const (\w+) = (\w+)\.(\w+);", line)
        if not m:
            continue
        name, lib, fn = m.groups()
        file = imports[lib]
        ln, params = find_fn(d, file, fn)
        row = dict(name=name, alias_line=n + 1, target=fn, file="src/Core/Tensor/TensorMath/" + file, line=ln,
                   params=params, kind="fn" if params is not None else "type", scope="out" if name in OUT_OF_SCOPE else "hot-path")
        if name in OUT_OF_SCOPE:
            row["why_out"] = OUT_OF_SCOPE[name]
        rows.append(row)
    # every tensMath.<name> that the generator's emitters and the hand-kept generated samples use
    emitted = {}
    for rel in ("src/codeGen/math_handler.zig", "src/codeGen/hardcoded/hardcoded_mnist8.zig", "src/codeGen/hardcoded/hardcoded_sentiment_it.zig",
                "src/codeGen/hardcoded/hardcoded_wakeWord.zig", "src/codeGen/test_mnist-1.zig"):
        path = os.path.join(ref, rel)
        if not os.path.exists(path):
            continue
        for i, line in enumerate(open(path).read().split("\n")):
            if line.strip().startswith("//"):
                continue
            for nm in re.findall(r"tensMath\.(\w+)", line):
                emitted.setdefault(nm, f"{rel}:{i + 1}")
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tensor_math_names.json")
    json.dump(dict(source="src/Core/Tensor/TensorMath/tensor_math_standard.zig", names=rows,
                   used_by_generated_code=[dict(name=k, first_use=v) for k, v in sorted(emitted.items())]), open(out, "w"), indent=1)
    print(len(rows), "names;", sum(r["scope"] == "hot-path" for r in rows), "on the inference path ->", out)


if __name__ == "__main__":
    main(sys.argv[1])
