#!/usr/bin/env python
"""Extracts the golden vectors that gorgonia's own tests hold for the hot path into JSON fixtures.

    python tests/golden/extract_goldens.py /path/to/gorgonia

It READS the Go test files as text (nothing of gorgonia is executed; there is no Go toolchain
here) and writes one JSON file per table next to this script. Only data is taken: the literal
inputs and expected outputs of the tables named below. The fixtures are committed; this script
is the record of where every number came from.

  binop.json           binOpTests                          op_math_test.go
  softmax_do.json      testCasesSoftMaxDo                  op_softmax_test.go
  maxpool_asym.json    TestMaxPool2D_asymmetricPadding     nn_test.go
  maxpool_basic.json   TestMaxPool                         nn_test.go
  conv_issue233.json   TestIssue233_F32 / _F64             known_issues_test.go
  leakyrelu.json       TestLeakyRelu                       nn_test.go
  byindices.json       TestByIndicesOpDo                   op_by_indices_test.go
  broadcast_add.json   broadcastAddTests                   operations_broadcast_test.go
  batchnorm.json       bnAllCases                          nn_amd64_test.go
  dropout.json         TestDropoutAll                      op_dropout_test.go
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
NUM = r"[-+]?(?:\d+\.?\d*(?:[eE][-+]?\d+)?|\.\d+(?:[eE][-+]?\d+)?)"


def strip_comments(src):
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return re.sub(r"//[^\n]*", "", src)


def balanced(src, start, open_ch, close_ch):
    """Index just past the bracket that closes the one at src[start]."""
    depth = 0
    for i in range(start, len(src)):
        if src[i] == open_ch:
            depth += 1
        elif src[i] == close_ch:
            depth -= 1
            if depth == 0:
                return i + 1
    raise ValueError("unbalanced")


def numbers(text):
    return [float(x) for x in re.findall(NUM, text)]


def region(src, start_marker, end_marker=None):
    a = src.index(start_marker)
    b = src.index(end_marker, a) if end_marker else len(src)
    return src[a:b]


def parse_value(expr):
    """tensor.New(...) / NewF64(x) / NewF32(x) -> dict(kind, dtype, shape, data)."""
    expr = expr.strip()
    m = re.match(r"NewF(64|32)\((" + NUM + r")\)", expr)
    if m:
        return {"kind": "scalar", "dtype": "float" + m.group(1), "shape": [], "data": [float(m.group(2))]}
    if not expr.startswith("tensor.New("):
        raise ValueError("cannot parse value: " + expr[:60])
    shape = None
    m = re.search(r"WithShape\(([^)]*)\)", expr)
    if m:
        shape = [int(v) for v in numbers(m.group(1))]
    m = re.search(r"WithBacking\(\s*\[\]\s*(float64|float32|int)\s*\{", expr)
    if m:
        end = balanced(expr, m.end() - 1, "{", "}")
        data = numbers(expr[m.end():end - 1])
        dtype = m.group(1)
    else:
        m = re.search(r"tensor\.Range\(\s*tensor\.(Float64|Float32)\s*,\s*(\d+)\s*,\s*(\d+)\s*\)", expr)
        if not m:
            raise ValueError("no backing: " + expr[:80])
        data = [float(v) for v in range(int(m.group(2)), int(m.group(3)))]
        dtype = m.group(1).lower()
    if shape is None:
        shape = [len(data)]
    return {"kind": "tensor", "dtype": dtype, "shape": shape, "data": data}


def values_in(src):
    """All tensor.New(...) / NewF64 / NewF32 expressions of a text, in order."""
    out = []
    for m in re.finditer(r"tensor\.New\(|NewF(?:64|32)\(", src):
        if out and m.start() < out[-1][1]:
            continue  # nested inside the previous one
        end = balanced(src, src.index("(", m.start()), "(", ")")
        out.append((m.start(), end))
    return [parse_value(src[a:b]) for a, b in out]


def top_level_blocks(src):
    """The {...} entries of a Go composite literal whose text starts at its opening brace."""
    blocks, i, depth = [], 0, 0
    start = None
    body_open = src.index("{")
    i = body_open + 1
    while i < len(src):
        ch = src[i]
        if ch == "{":
            if depth == 0:
                start = i
            depth += 1
        elif ch == "}":
            if depth == 0:
                break
            depth -= 1
            if depth == 0:
                blocks.append(src[start:i + 1])
        i += 1
    return blocks


def field(block, name, pattern):
    m = re.search(name + r"\s*:\s*" + pattern, block)
    return m.group(1) if m else None


def extract_binop(root):
    src = strip_comments(open(os.path.join(root, "op_math_test.go")).read())
    table = region(src, "var binOpTests = []binOpTest", "\nfunc ")
    table = table[table.index("=") + 1:]
    table = table[table.index("]binOpTest") + len("]binOpTest"):]
    cases = []
    for blk in top_level_blocks(table):
        m = re.match(r"\{\s*([A-Za-z]+)\s*,", blk)
        if m:
            op = m.group(1)
        elif "BatchedMatMul" in blk:
            op = "BatchedMatMul"
        else:
            continue
        vals = values_in(blk)
        if len(vals) < 5:
            continue
        sm = re.search(r"tensor\.Shape\{([^}]*)\}\s*,?\s*\}\s*$", blk)
        shape = [int(v) for v in numbers(sm.group(1))] if sm else []
        cases.append({"op": op, "a": vals[0], "b": vals[1], "correct": vals[2], "deriv_a": vals[3],
                      "deriv_b": vals[4], "correct_shape": shape})
    return {"source": "op_math_test.go: binOpTests", "cases": cases}


def extract_softmax(root):
    src = strip_comments(open(os.path.join(root, "op_softmax_test.go")).read())
    table = region(src, "var testCasesSoftMaxDo", "\nfunc ")
    table = table[table.index("}{") + 1:]
    cases = []
    for blk in top_level_blocks(table):
        arrays = []
        for m in re.finditer(r"\[\]float64\s*\{", blk):
            end = balanced(blk, m.end() - 1, "{", "}")
            arrays.append(numbers(blk[m.end():end - 1]))
        shape = [int(v) for v in numbers(re.search(r"tensor\.Shape\{([^}]*)\}", blk).group(1))]
        cases.append({"input": arrays[0], "shape": shape, "expected": arrays[1]})
    return {"source": "op_softmax_test.go: testCasesSoftMaxDo (softmax along the last axis)", "cases": cases}


def extract_maxpool_asym(root):
    src = strip_comments(open(os.path.join(root, "nn_test.go")).read())
    fn = region(src, "func TestMaxPool2D_asymmetricPadding", "\nfunc ")
    vals = values_in(fn)
    cases = [{"input": vals[i], "output": vals[i + 1]} for i in range(0, len(vals) - 1, 2)]
    return {"source": "nn_test.go: TestMaxPool2D_asymmetricPadding", "kernel": [2, 2], "pad": [1, 0, 1, 0],
            "stride": [1, 1], "cases": cases}


def extract_maxpool_basic(root):
    src = strip_comments(open(os.path.join(root, "nn_test.go")).read())
    fn = region(src, "func TestMaxPool(t", "\nfunc ")
    table = fn[fn.index("}{") + 1:]
    cases = []
    for blk in top_level_blocks(table):
        if "input" not in blk:
            continue
        cases.append({
            "input": values_in(blk)[0],
            "kernel": [int(v) for v in numbers(field(blk, "kernelSize", r"\[\]int\{([^}]*)\}"))],
            "pad": [int(v) for v in numbers(field(blk, "pad", r"\[\]int\{([^}]*)\}"))],
            "stride": [int(v) for v in numbers(field(blk, "stride", r"\[\]int\{([^}]*)\}"))],
            "expected": numbers(field(blk, "expectedOutput", r"\[\]float64\{([^}]*)\}")),
            "expected_shape": [int(v) for v in numbers(field(blk, "expectedShape", r"tensor\.Shape\{([^}]*)\}"))],
        })
    return {"source": "nn_test.go: TestMaxPool", "cases": cases}


def extract_conv(root):
    src = strip_comments(open(os.path.join(root, "known_issues_test.go")).read())
    cases = []
    for name in ("TestIssue233_F32", "TestIssue233_F64"):
        fn = region(src, "func " + name, "\nfunc ")
        vals = values_in(fn)
        m = re.search(r"correct\s*:=\s*\[\]float(?:32|64)\s*\{", fn)
        end = balanced(fn, m.end() - 1, "{", "}")
        cases.append({"name": name, "x": vals[0], "w": vals[1], "kernel": [3, 3], "pad": [1, 1], "stride": [1, 1],
                      "dilation": [1, 1], "correct": numbers(fn[m.end():end - 1])})
    return {"source": "known_issues_test.go: TestIssue233_F32 / TestIssue233_F64 (Conv2d 3x3, pad 1)", "cases": cases}


def extract_leakyrelu(root):
    src = strip_comments(open(os.path.join(root, "nn_test.go")).read())
    fn = region(src, "func TestLeakyRelu", "\nfunc ")
    table = fn[fn.index("}{") + 1:]
    cases = []
    for blk in top_level_blocks(table):
        vals = values_in(blk)
        if len(vals) != 2:
            continue
        cases.append({"alpha": float(field(blk, "alpha", "(" + NUM + ")")), "x": vals[0], "y": vals[1]})
    return {"source": "nn_test.go: TestLeakyRelu (compared there with InDeltaSlice 1e-6)", "cases": cases}


def extract_byindices(root):
    src = strip_comments(open(os.path.join(root, "op_by_indices_test.go")).read())
    fn = region(src, "func TestByIndicesOpDo", "\nfunc ")
    table = fn[fn.index("}{") + 1:]
    cases = []
    for blk in top_level_blocks(table):
        vals = values_in(blk)
        if len(vals) != 2:
            continue
        cases.append({"input": vals[0], "indices": vals[1], "axis": int(field(blk, "axis", r"(\d+)")),
                      "expected": numbers(field(blk, "expectedOutput", r"\[\]float64\{([^}]*)\}")),
                      "expected_shape": [int(v) for v in numbers(field(blk, "expectedShape",
                                                                         r"tensor\.Shape\{([^}]*)\}"))]})
    return {"source": "op_by_indices_test.go: TestByIndicesOpDo", "cases": cases}


def extract_broadcast(root):
    src = strip_comments(open(os.path.join(root, "operations_broadcast_test.go")).read())
    table = region(src, "var broadcastAddTests", "\nvar ")
    table = table[table.index("]broadcastOpTest") + len("]broadcastOpTest"):]
    cases = []
    for blk in top_level_blocks(table):
        if re.search(r"err\s*:\s*true", blk):
            continue
        vals = values_in(blk)
        if len(vals) != 3:
            continue
        left = field(blk, "left", r"\[\]byte\{([^}]*)\}")
        right = field(blk, "right", r"\[\]byte\{([^}]*)\}")
        cases.append({"name": field(blk, "name", r'"([^"]*)"'), "a": vals[0], "b": vals[1], "ab": vals[2],
                      "left": [int(v) for v in numbers(left)] if left else [],
                      "right": [int(v) for v in numbers(right)] if right else []})
    return {"source": "operations_broadcast_test.go: broadcastAddTests (left/right = axes along which that "
                      "operand is repeated)", "cases": cases}


def extract_batchnorm(root):
    """bnAllCases (nn_amd64_test.go:8-...): input / scale / bias initialisers and, after ONE training run from
    running mean 0 and running variance 1, the running statistics and the output of
    ((BatchNorm(x) * scale + bias) reshaped to (B, F)) x fcWeight^T, fcWeight (B, F) filled by ScaleInit."""
    src = strip_comments(open(os.path.join(root, "nn_amd64_test.go")).read())
    table = src[src.index("}{", src.index("var bnAllCases")) + 1:]

    def init(expr):
        expr = expr.strip()
        m = re.match(r"RangedFromWithStep\((" + NUM + r")\s*,\s*(" + NUM + r")\)", expr)
        if m:
            return {"kind": "ranged", "start": float(m.group(1)), "step": float(m.group(2))}
        if expr.startswith("Ones()"):
            return {"kind": "ones"}
        if expr.startswith("Zeroes()"):
            return {"kind": "zeroes"}
        m = re.match(r"\[\]float(?:32|64)\{([^}]*)\}", expr)
        if m:
            return {"kind": "literal", "data": numbers(m.group(1))}
        raise ValueError("cannot parse initialiser: " + expr[:60])

    cases = []
    for blk in top_level_blocks(table):
        if "ExpectedTrainResult" not in blk:
            continue
        def arr(name):
            return numbers(field(blk, name, r"\[\]float(?:32|64)\{([^}]*)\}"))
        cases.append({
            "desc": field(blk, "desc", r'"([^"]*)"'),
            "dtype": "float32" if "tensor.Float32" in field(blk, "Dtype", r"(tensor\.Float\d+)") else "float64",
            "x": init(field(blk, "X", r"((?:RangedFromWithStep\([^)]*\))|(?:\[\]float(?:32|64)\{[^}]*\}))")),
            "x_shape": [int(v) for v in numbers(field(blk, "XShape", r"tensor\.Shape\{([^}]*)\}"))],
            "scale": init(field(blk, "ScaleInit", r"((?:RangedFromWithStep\([^)]*\))|(?:Ones\(\))|(?:Zeroes\(\)))")),
            "bias": init(field(blk, "BiasInit", r"((?:RangedFromWithStep\([^)]*\))|(?:Ones\(\))|(?:Zeroes\(\)))")),
            "train_result": arr("ExpectedTrainResult"),
            "running_mean": arr("ExpectedMean"),
            "running_var": arr("ExpectedVariance"),
        })
    return {"source": "nn_amd64_test.go: bnAllCases, checked there with dawson.AllClose (nn_test.go:319-440); momentum 0.9, "
                      "epsilon 1e-5", "cases": cases}


def extract_dropout(root):
    """TestDropoutAll (op_dropout_test.go:14-68): x = ones(5), an injected generator that cycles through
    `rand`, cost = Mean(y); expected y, dcost/dy and dcost/dx."""
    src = strip_comments(open(os.path.join(root, "op_dropout_test.go")).read())
    table = region(src, "var tests = []struct", "for _, tt := range tests")
    table = table[table.index("}{") + 1:]
    cases = []
    for blk in top_level_blocks(table):
        m = re.match(r"\{\s*(Float64|Float32)\s*,\s*(" + NUM + r")\s*,(.*)\}\s*$", blk.strip(), flags=re.S)
        if not m:
            continue
        lists = re.findall(r"\[\]float(?:32|64)\{([^}]*)\}", m.group(3))
        if len(lists) != 4:
            raise ValueError("dropout case with %d lists" % len(lists))
        cases.append({"dtype": m.group(1).lower(), "prob": float(m.group(2)), "rand": numbers(lists[0]),
                      "y": numbers(lists[1]), "y_grad": numbers(lists[2]), "x_grad": numbers(lists[3])})
    return {"source": "op_dropout_test.go: TestDropoutAll; x = Ones() of shape (5), cost = Mean(y)", "cases": cases}


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: extract_goldens.py <path to a gorgonia checkout>")
    root = sys.argv[1]
    out = {
        "binop.json": extract_binop(root),
        "softmax_do.json": extract_softmax(root),
        "maxpool_asym.json": extract_maxpool_asym(root),
        "maxpool_basic.json": extract_maxpool_basic(root),
        "conv_issue233.json": extract_conv(root),
        "leakyrelu.json": extract_leakyrelu(root),
        "byindices.json": extract_byindices(root),
        "broadcast_add.json": extract_broadcast(root),
        "batchnorm.json": extract_batchnorm(root),
        "dropout.json": extract_dropout(root),
    }
    for name, doc in out.items():
        with open(os.path.join(HERE, name), "w") as f:
            json.dump(doc, f, separators=(",", ":"))
        print(f"{name}: {len(doc['cases'])} cases, {os.path.getsize(os.path.join(HERE, name))} bytes")


if __name__ == "__main__":
    main()
