"""The three descriptions of the C ABI agree: include/alpha_cuda.h (the source), the bun:ffi
table ts/ffi.ts that a TypeScript host binds (generated from the header; it cannot be run here,
so it is at least checked), the ctypes table alpha2_b200/_lib.py that every test goes through,
and the excerpts shown in INTEGRATION.md.  Name, arity and every scalar type are compared: an
entry bound with one argument too few passes garbage for the missing one."""
import ctypes as C
import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "ts"))
import gen_ffi  # noqa: E402

from alpha2_b200 import _lib as L  # noqa: E402


def _parse_ts(text: str) -> dict:
    out = {}
    for m in re.finditer(r"(alpha_[a-z0-9_]+):\s*\{\s*args:\s*\[([^\]]*)\],\s*returns:\s*(?:T|FFIType)\.(\w+)\s*\}", text, flags=re.S):
        args = [a.strip().split(".")[-1] for a in m.group(2).split(",") if a.strip()]
        out[m.group(1)] = (m.group(3), args)
    return out


def _ctypes_to_ffi(t, result: bool = False) -> str:
    if t in (C.c_void_p, C.c_char_p) or (isinstance(t, type) and issubclass(t, C._Pointer)):
        return "cstring" if (t is C.c_char_p and result) else "ptr"     # a string argument is a plain pointer
    return {C.c_int: "i32", C.c_int32: "i32", C.c_uint32: "u32", C.c_int64: "i64", C.c_uint64: "u64",
            C.c_size_t: "u64", C.c_float: "f32", C.c_double: "f64"}[t]


def test_generated_ts_table_is_current_and_matches_the_header():
    hdr = gen_ffi.parse_header()
    assert len(hdr) > 80
    committed = open(os.path.join(ROOT, "ts", "ffi.ts")).read()
    assert committed == gen_ffi.render(hdr), "ts/ffi.ts is stale: run python ts/gen_ffi.py"
    ts = _parse_ts(committed)
    assert set(ts) == set(hdr)
    for name, (ret, types, _) in hdr.items():
        assert ts[name] == (ret, types), name


def test_ctypes_table_matches_the_header():
    hdr = gen_ffi.parse_header()
    table = {n: ("i32", a) for n, a in L.SIGNATURES.items()}
    table.update({n: (_ctypes_to_ffi(r, result=True), a) for n, (a, r) in L._OTHER_RESTYPE.items()})
    assert set(table) == set(hdr), sorted(set(table) ^ set(hdr))
    for name, (ret, types, names) in hdr.items():
        got_ret, got_args = table[name]
        assert got_ret == ret, name
        assert [_ctypes_to_ffi(a) for a in got_args] == types, (name, names)


def test_integration_md_excerpts_match_the_header():
    hdr = gen_ffi.parse_header()
    doc = _parse_ts(open(os.path.join(ROOT, "INTEGRATION.md")).read())
    assert len(doc) >= 20
    for name, (ret, args) in doc.items():
        assert name in hdr, name
        assert (ret, args) == (hdr[name][0], hdr[name][1]), name


def _calls(text: str):
    """(name, number of top-level arguments) of every `C.alpha_*( ... )` call in a TypeScript text."""
    out = []
    for m in re.finditer(r"\bC\.(alpha_[a-z0-9_]+)\(", text):
        i, depth, args, cur = m.end(), 1, 0, ""
        while depth:
            ch = text[i]
            if ch in "([{":
                depth += 1
            elif ch in ")]}":
                depth -= 1
                if depth == 0:
                    break
            elif ch == "," and depth == 1:
                args += 1
                cur = ""
                i += 1
                continue
            cur += ch
            i += 1
        out.append((m.group(1), args + (1 if cur.strip() else 0)))
    return out


# every method of the reference's Backend interface (packages/core/src/interfaces.ts:38-151)
BACKEND_METHODS = """zeros ones full randn fromArray add sub mul div matmul sum mean neg exp log sqrt pow scale clamp
embedding layerNorm gelu relu silu softmax logSoftmax crossEntropy reshape transpose slice cat argmax topk gather clone
equal allClose causalMask maskedFill geluBackward reluBackward siluBackward siluMul siluMulBackward clampBackward
layerNormBackward crossEntropyBackward embeddingBackward softCap softCapBackward residualDropoutAdd matmulTransposed
matmulTransposedA addInplace scaleInplace sliceQkv scatterSlice dropoutMask flashAttention flashAttentionBackward
broadcast castDtype sumOfSquares totalSumOfSquares checkFinite adamwStep""".split()
# what the trainer and the CLI probe by duck typing (trainer.ts:623-641,757-841,998-1044; train.ts:284-318)
PROBED = "releaseGpuTensor flush syncGpu purgeBufferPools gpuMemStats resetStepOps gpuOpsThisStep getDeviceInfo smokeTest setMinGpuSize coopMatmulPaused getMatmulCoopStats".split()


def test_typescript_backend_calls_the_abi_with_the_declared_arity_and_covers_the_interface():
    hdr = gen_ffi.parse_header()
    text = open(os.path.join(ROOT, "ts", "backend.ts")).read()
    calls = _calls(text)
    assert len(calls) > 50
    for name, n in calls:
        assert name in hdr, name
        assert n == len(hdr[name][1]), (name, n, hdr[name][2])
    for meth in BACKEND_METHODS + PROBED:
        assert re.search(r"\n  (?:readonly |get |private )?%s\b" % meth, text), meth
