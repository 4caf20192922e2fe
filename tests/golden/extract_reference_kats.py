#!/usr/bin/env python3
"""Extract the reference's own known-answer vectors for the MobileNet inference path.

Reads the literal arrays inside tfjs-core's jasmine spec files (as text; nothing is
executed) and writes them to ``reference_kats.json`` next to this script.  Run in a
container where the reference checkout is mounted::

    python tests/golden/extract_reference_kats.py <path to the tfjs checkout>

Each case records the spec file and the line of its ``it(...)`` so a reader can find it.
Operands are located inside the spec body by element count: ``sized(n, k)`` is the k-th
numeric array literal with exactly n elements, ``last()`` the final literal (the expected
values in every spec used here).  Op parameters (shapes, strides, pads) are restated from
the spec text next to each case.
"""
import json
import math
import os
import re
import sys

_NUM = r"-?(?:\d+\.?\d*|\.\d+)(?:e-?\d+)?|NaN|[-+]?Infinity|\+\d+"
NUM_ARRAY = re.compile(r"\[\s*(?:(?:" + _NUM + r")\s*,?\s*)+\]")


def spec_block(root, rel, name, occurrence=0):
    text = open(os.path.join(root, rel)).read()
    pat = re.compile(r"\n\s*it\(\s*\n?\s*'" + re.escape(name) + r"'")
    ms = list(pat.finditer(text))
    if len(ms) <= occurrence:
        raise KeyError(f"{rel}: spec {name!r} occurrence {occurrence} not found")
    start = ms[occurrence].start() + 1
    nxt = re.compile(r"\n\s*(?:it|xit|describeWithFlags|describe)\(").search(
        text, ms[occurrence].end())
    end = nxt.start() if nxt else len(text)
    # skip the spec title itself: titles such as 'x=[2,2,1] f=[1,1,1,2]' contain brackets
    return text[ms[occurrence].end():end], text.count("\n", 0, start) + 1


def parse_num(tok):
    tok = tok.strip()
    if tok in ("NaN", "Infinity", "-Infinity", "+Infinity"):
        return tok.lstrip("+")
    return float(tok)


class Lits:
    def __init__(self, block):
        self.items = []
        for m in NUM_ARRAY.finditer(block):
            body = m.group(0)[1:-1]
            self.items.append([parse_num(t) for t in body.split(",") if t.strip()])

    def sized(self, n, k=0):
        hits = [l for l in self.items if len(l) == n]
        return hits[k]

    def last(self):
        return self.items[-1]

    def first(self):
        return self.items[0]


def prod(shape):
    return int(math.prod(shape))


CASES = []


def case(kind, rel, name, build, occurrence=0):
    CASES.append((kind, rel, name, build, occurrence))


OPS = "tfjs-core/src/ops/"
FUSED = OPS + "fused_test.ts"

# ---- fused matMul (ops/fused_test.ts 'fused matmul') ---------------------------------------
_A, _B = [2, 3], [3, 2]


def fm(name, a_shape=_A, b_shape=_B, **kw):
    def build(l):
        d = dict(a=l.sized(prod(a_shape), 0), a_shape=a_shape,
                 b=l.sized(prod(b_shape), 1 if prod(a_shape) == prod(b_shape) else 0),
                 b_shape=b_shape, expected=l.last())
        for k, v in kw.items():
            d[k] = v(l) if callable(v) else v
        return d
    case("fused_matmul", FUSED, name, build)


fm("A x B")
fm("A x B with relu", activation="relu")
fm("A x B with prelu", activation="prelu", prelu=[0.5, 0.5], prelu_shape=[1, 2])
fm("A x B with relu transpose", b_shape=[2, 3], transpose_b=True, activation="relu")
fm("A x B with relu and bias", activation="relu", bias=[1.0, 1.0, 1.0, 1.0], bias_shape=[2, 2])
fm("A x B with relu and broadcasted bias", activation="relu", bias=[1.0, 1.0], bias_shape=[2])
fm("A x B with relu and broadcasted bias different rank", a_shape=[2, 2, 3], b_shape=[2, 3, 2],
   activation="relu", bias=[1.0, 2.0], bias_shape=[1, 2])
fm("A x B with bias only", bias=[1.0, 1.0, 1.0, 1.0], bias_shape=[2, 2])

# ---- fused conv2d (ops/fused_test.ts 'fused conv2d') ---------------------------------------


def conv(kind, rel, name, x_shape, w_shape, strides, pad, xk=0, wk=0, occurrence=0, **kw):
    def build(l):
        d = dict(x=l.sized(prod(x_shape), xk), x_shape=x_shape,
                 w=l.sized(prod(w_shape), wk), w_shape=w_shape, strides=strides, pad=pad,
                 expected=l.last())
        for k, v in kw.items():
            d[k] = v(l) if callable(v) else v
        return d
    case(kind, rel, name, build, occurrence)


conv("fused_conv2d", FUSED, "basic", [2, 2, 2, 2], [1, 1, 2, 2], 1, 0, xk=0, wk=0)
conv("fused_conv2d", FUSED, "basic with relu", [2, 2, 2, 2], [1, 1, 2, 2], 1, 0,
     activation="relu")
conv("fused_conv2d", FUSED, "basic with prelu", [2, 2, 2, 2], [1, 1, 2, 2], 1, 0,
     activation="prelu", prelu=[0.25, 0.75], prelu_shape=[1, 1, 2])
conv("fused_conv2d", FUSED, "basic with bias and relu", [2, 2, 2, 2], [1, 1, 2, 2], 1, 0,
     activation="relu", bias=[5.0], bias_shape=[])
IM = dict(x_shape=[1, 4, 4, 1], w_shape=[1, 1, 1, 3])
conv("fused_conv2d", FUSED, "im2row", strides=2, pad="same", **IM)
conv("fused_conv2d", FUSED, "im2row with relu", strides=2, pad="same", activation="relu", **IM)
conv("fused_conv2d", FUSED, "im2row with prelu", strides=2, pad="same", activation="prelu",
     prelu=[0.5], prelu_shape=[1, 1, 1], **IM)
conv("fused_conv2d", FUSED, "pointwise with prelu", strides=1, pad="same", activation="prelu",
     prelu=[0.5], prelu_shape=[1, 1, 1], **IM)
conv("fused_conv2d", FUSED, "im2row with bias and relu", strides=2, pad="same",
     activation="relu", bias=[5.0], bias_shape=[], **IM)

# ---- conv2d (ops/conv2d_test.ts) -----------------------------------------------------------
C2 = OPS + "conv2d_test.ts"
conv("conv2d", C2, "x=[1,4,4,1] f=[1,1,1,3] s=2 d=1 p=same", [1, 4, 4, 1], [1, 1, 1, 3], 2, "same")
conv("conv2d", C2, "x=[2,2,1] f=[1,1,1,2] s=1 d=1 p=0", [1, 2, 2, 1], [1, 1, 1, 1], 1, 0)
conv("conv2d", C2, "x=[3,3,2] f=[2,2,2,1] s=1 d=1 p=valid", [1, 3, 3, 2], [2, 2, 2, 1], 1, "valid")
conv("conv2d", C2, "x=[2,2,2,1] f=[1,1,1,1] s=1 d=1 p=0", [2, 2, 2, 1], [1, 1, 1, 1], 1, 0)
conv("conv2d", C2, "x=[4,2,1] f=[4,2,1,1] s=1 d=1 p=same", [1, 4, 2, 1], [4, 2, 1, 1], 1, "same",
     xk=0, wk=1)
conv("conv2d", C2, "x=[2,2,1] f=[2,2,1,1] s=1 d=1 p=same", [1, 2, 2, 1], [2, 2, 1, 1], 1, "same",
     xk=0, wk=1)
conv("conv2d", C2, "x=[2,2,1] f=[2,2,1,1] s=1 d=1 p=0", [1, 2, 2, 1], [2, 2, 1, 1], 1, 0,
     xk=0, wk=1)
# dilation 2 must equal the zero-stuffed 3x3 filter at dilation 1 (equivalence spec)
conv("conv2d_dilation_equiv", C2, "x=[4,4,1] f=[2,2,1,1] s=1 d=2 p=0", [1, 4, 4, 1],
     [2, 2, 1, 1], 1, 0, dilation=2, w_dilated=lambda l: l.sized(9), w_dilated_shape=[3, 3, 1, 1],
     expected=None)
# generateCaseInputs (conv2d_test.ts:23-35): input = 1..n, filter = 1..m
case("conv2d", C2, "x=[1,3,6,1] f=[2,2,1,1] s=[1,2] d=1 p=valid",
     lambda l: dict(x=[float(i + 1) for i in range(18)], x_shape=[1, 3, 6, 1],
                    w=[1.0, 2.0, 3.0, 4.0], w_shape=[2, 2, 1, 1], strides=[1, 2], pad="valid",
                    expected=l.last()))

# ---- depthwiseConv2D (ops/conv2d_depthwise_test.ts) ----------------------------------------
DW = OPS + "conv2d_depthwise_test.ts"
conv("depthwise", DW, "input=1x3x3x1,f=2,s=1,d=1,p=valid,chMul=1", [1, 3, 3, 1], [2, 2, 1, 1], 1,
     "valid", wk=0)
conv("depthwise", DW, "input=1x5x5x1,f=3,s=1,d=1,p=valid,chMul=1", [1, 5, 5, 1], [3, 3, 1, 1], 1,
     "valid", wk=0)
conv("depthwise_dilation_equiv", DW, "input=1x3x3x1,f=2,s=1,d=2,p=valid,chMul=1", [1, 3, 3, 1],
     [2, 2, 1, 1], 1, "valid", dilation=2, w_dilated=lambda l: l.sized(9, 1),
     w_dilated_shape=[3, 3, 1, 1], expected=None)
conv("depthwise_dilation_equiv", DW, "input=1x5x5x1,f=3,s=1,d=2,p=valid,chMul=1", [1, 5, 5, 1],
     [3, 3, 1, 1], 1, "valid", dilation=2, w_dilated=lambda l: l.sized(25, 1),
     w_dilated_shape=[5, 5, 1, 1], expected=None)
conv("depthwise", DW, "input=1x3x3x2,f=2,s=1,d=1,p=same,chMul=1", [1, 3, 3, 2], [2, 2, 2, 1], 1,
     "same")
conv("depthwise", DW, "input=1x5x5x1,f=3,s=1,d=1,p=same,chMul=1", [1, 5, 5, 1], [3, 3, 1, 1], 1,
     "same")
conv("depthwise", DW, "input=1x3x3x2,f=2,s=1,p=same,chMul=2", [1, 3, 3, 2], [2, 2, 2, 2], 1,
     "same")
conv("depthwise", DW, "input=2x3x3x2,f=2,s=1,p=same,chMul=2", [2, 3, 3, 2], [2, 2, 2, 2], 1,
     "same")

# ---- separableConv2d = depthwise then 1x1 conv2d (ops/conv2d_separable_test.ts) ------------
SEP = OPS + "conv2d_separable_test.ts"


def sep(name, x_shape, dw_shape, pw_shape, strides, pad, pwk=0):
    def build(l):
        return dict(x=l.sized(prod(x_shape)), x_shape=x_shape, dw=l.sized(prod(dw_shape)),
                    dw_shape=dw_shape, pw=l.sized(prod(pw_shape), pwk), pw_shape=pw_shape,
                    strides=strides, pad=pad, expected=l.last() if len(l.last()) > 4
                    else l.items[-2])
    case("separable", SEP, name, build)


sep("input=1x4x4x1,f=2,s=2,d=1,p=valid,chMul=1,outDepth=2", [1, 4, 4, 1], [2, 2, 1, 1],
    [1, 1, 1, 2], 2, "valid", pwk=1)  # the first 2-element literal is the stride [2, 2]
sep("input=2x4x4x1,f=2,s=2,d=1,p=valid,chMul=1,outDepth=2", [2, 4, 4, 1], [2, 2, 1, 1],
    [1, 1, 1, 2], 2, "valid", pwk=1)  # the first 2-element literal is the stride [2, 2]
sep("input=1x4x4x2,f=2,s=2,d=1,p=valid,chMul=1,outDepth=2", [1, 4, 4, 2], [2, 2, 2, 1],
    [1, 1, 2, 2], 2, "valid")

# ---- matMul (ops/matmul_test.ts) -----------------------------------------------------------
MM = OPS + "matmul_test.ts"


def mm(name, a_shape, b_shape, ta=False, tb=False, occurrence=0):
    def build(l):
        same = prod(a_shape) == prod(b_shape)
        return dict(a=l.sized(prod(a_shape), 0), a_shape=a_shape,
                    b=l.sized(prod(b_shape), 1 if same else 0), b_shape=b_shape,
                    transpose_a=ta, transpose_b=tb, expected=l.last())
    case("matmul", MM, name, build, occurrence)


mm("A x B", [2, 3], [3, 2])
mm("[8,4]x[4,8]", [8, 4], [4, 8])
mm("A x B^t", [2, 3], [2, 3], tb=True)
mm("A^t x B", [2, 3], [2, 3], ta=True)
mm("A^t x B^t", [3, 2], [2, 3], ta=True, tb=True)
mm("A x B", [5, 2, 3], [5, 3, 2], occurrence=1)
mm("A x B^t", [5, 2, 3], [5, 2, 3], tb=True, occurrence=1)
mm("A^t x B", [5, 2, 3], [5, 2, 3], ta=True, occurrence=1)
mm("A^t x B^t", [5, 3, 2], [5, 2, 3], ta=True, tb=True, occurrence=1)
case("matmul", MM, "Matrix * vector propagates NaNs",
     lambda l: dict(a=[1.0, 2.0, 3.0, 4.0], a_shape=[2, 2], b=[2.0, "NaN"], b_shape=[2, 1],
                    transpose_a=False, transpose_b=False, expected=["NaN", "NaN"]))

# The only known-answer vector larger than one tile: tfjs-webgpu/src/matmul_test.ts
case("matmul", "tfjs-webgpu/src/matmul_test.ts", "matMul A x B multiple tiles",
     lambda l: dict(a=l.sized(65 * 67), a_shape=[65, 67], b=l.sized(67 * 66), b_shape=[67, 66],
                    transpose_a=False, transpose_b=False, expected=l.sized(65 * 66)))

# ---- pooling (ops/pool_test.ts) ------------------------------------------------------------
PL = OPS + "pool_test.ts"


def pool(kind, name, x_shape, f, s, pad, occurrence=0, rounding=None, shape_only=False):
    def build(l):
        d = dict(pool=kind, x=l.sized(prod(x_shape), 0), x_shape=x_shape, filter=f, strides=s,
                 pad=pad, rounding=rounding)
        if shape_only:
            d["expected_shape"] = [1, 2, 2, 3]
        else:
            d["expected"] = l.last()
        return d
    case("pool", PL, name, build, occurrence)


pool("max", "x=[1,1,1] f=[1,1] s=1 [0] => [0]", [1, 1, 1, 1], 1, 1, 0)
pool("max", "x=[3,3,1] f=[2,2] s=1, p=0", [1, 3, 3, 1], 2, 1, 0)
pool("max", "x=[3,3,1] f=[2,2] s=1 p=same", [1, 3, 3, 1], 2, 1, "same")
pool("max", "x=[2,3,3,1] f=[2,2] s=1", [2, 3, 3, 1], 2, 1, 0)
pool("max", "[x=[3,3,1] f=[2,2] s=1 ignores NaNs", [1, 3, 3, 1], 2, 1, 0)
pool("max", "x=[3,3,2] f=[2,2] s=1", [1, 3, 3, 2], 2, 1, 0)
pool("max", "x=[4,4,1] f=[2,2] s=2", [1, 4, 4, 1], 2, 2, 0)
pool("max", "x=[2,2,1] f=[2,2] s=1 p=same", [1, 2, 2, 1], 2, 1, "same")
pool("max", "x=[2,2,3] f=[1,1] s=2 p=1 dimRoundingMode=floor", [1, 2, 2, 3], 1, 2, 1,
     rounding="floor", shape_only=True)
pool("avg", "x=[1,1,1] f=[1,1] s=1 [0] => [0]", [1, 1, 1, 1], 1, 1, 0, occurrence=1)
pool("avg", "x=[3,3,1] f=[2,2] s=1", [1, 3, 3, 1], 2, 1, 0)
pool("avg", "x=[2,3,3,1] f=[2,2], s=1", [2, 3, 3, 1], 2, 1, 0)
pool("avg", "x=[3,3,1] f=[2,2] s=1 propagates NaNs", [1, 3, 3, 1], 2, 1, 0)
pool("avg", "x=[3,3,2] f=[2,2] s=1", [1, 3, 3, 2], 2, 1, 0, occurrence=1)
pool("avg", "x=[4,4,1] f=[2,2] s=2", [1, 4, 4, 1], 2, 2, 0, occurrence=1)
pool("avg", "x=[2,2,1] f=[2,2] s=1 p=same", [1, 2, 2, 1], 2, 1, "same", occurrence=1)
pool("avg", "x=[2,2,3] f=[1,1] s=2 p=1 dimRoundingMode=floor", [1, 2, 2, 3], 1, 2, 1,
     occurrence=1, rounding="floor", shape_only=True)

# ---- softmax (ops/softmax_test.ts) ---------------------------------------------------------
SM = OPS + "softmax_test.ts"


def sm(name, shape):
    case("softmax", SM, name,
         lambda l: dict(x=l.sized(prod(shape), 0), x_shape=shape, expected=l.last()))


sm("regular test", [3])
sm("overflow", [2])
sm("underflow", [2])
case("softmax", SM, "Huge difference between probabilities",
     lambda l: dict(x=[-1000.0, 1000.0], x_shape=[2], expected=[0.0, 1.0]))
sm("Propagates NaNs", [3])
case("softmax", SM, "2D, dim=1",
     lambda l: dict(x=l.sized(3, 0) + l.sized(3, 1), x_shape=[2, 3], expected=l.last()))

# ---- clipByValue (ops/unary_ops_test.ts 'clip') --------------------------------------------
UN = OPS + "unary_ops_test.ts"
case("clip", UN, "basic",
     lambda l: dict(x=l.sized(6, 0), min=-1.0, max=50.0, expected=l.last()))
case("clip", UN, "propagates NaNs",
     lambda l: dict(x=l.sized(7, 0), min=-1.0, max=50.0, expected=l.last()), occurrence=None)

# ---- uint8 weight dequantisation (io/io_utils_test.ts) -------------------------------------
case("dequant_u8", "tfjs-core/src/io/io_utils_test.ts", "support quantization uint8 weights",
     lambda l: dict(q=[0, 48, 255], scale=0.1, min=-1.0, expected=l.sized(3, 0)))


def find_clip_occurrence(root, rel, name):
    """unary_ops_test.ts has many specs called 'basic'/'propagates NaNs'; take the one whose
    body calls tf.clipByValue."""
    text = open(os.path.join(root, rel)).read()
    pat = re.compile(r"\n\s*it\(\s*'" + re.escape(name) + r"'")
    for i, _ in enumerate(pat.finditer(text)):
        block, _ = spec_block(root, rel, name, i)
        if "clipByValue" in block:
            return i
    raise KeyError(name)


def main():
    root = sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else os.environ.get("TFJS_REFERENCE", "reference")
    out = []
    for kind, rel, name, build, occ in CASES:
        if kind == "clip":
            occ = find_clip_occurrence(root, rel, name)
        block, line = spec_block(root, rel, name, occ)
        rec = dict(kind=kind, source=f"{rel}:{line}", name=name)
        rec.update(build(Lits(block)))
        out.append(rec)
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "reference_kats.json"), "w") as f:
        f.write("[\n" + ",\n".join(json.dumps(r, separators=(",", ":")) for r in out) + "\n]\n")
    print(f"wrote {len(out)} cases")


if __name__ == "__main__":
    main()
