"""Transcribes the reference's quantisation known-answer tests into a JSON fixture.

The reference is Java and cannot be executed in this build environment, so the
vectors are read out of its test sources as text:

  node/src/test/java/cab/ml/juno/node/GgufReaderTest.java
      f16ToF32 exact values (:35-46), Q6_K golden block + 14 expected outputs (:60-105),
      Q6_K range block (:107-125), Q4_K all-zero (:334-358), Q4_K nibble split (:360-382),
      Q8_0 0.5*i block (:634-656)
  node/src/test/java/cab/ml/juno/node/PhiQuantizedMatVecTest.java
      Q4_K one-block dot (:69-112), Q4_K three-row range (:121-166, fillQ4KBlock :298-314),
      Q6_K golden-block dot (:199-238)

Usage:  python tests/golden/make_quant_known_answers.py /path/to/reference
Writes tests/golden/quant_known_answers.json next to this script.
"""
import json
import os
import re
import sys


def java_bytes(src: str, decl: str, start: int = 0):
    """Parse `byte[] <decl> = { ... };` after offset `start` into a list of 0..255 ints."""
    m = re.compile(r"byte\[\]\s+" + re.escape(decl) + r"\s*=\s*\{([^}]*)\}", re.S).search(src, start)
    vals = [int(v) for v in re.findall(r"-?\d+", m.group(1))]
    return [v & 0xFF for v in vals], m.end()


def main(ref_root: str):
    node_test = os.path.join(ref_root, "node/src/test/java/cab/ml/juno/node")
    src = open(os.path.join(node_test, "GgufReaderTest.java"), encoding="utf-8").read()

    out = {"source": "ml-cab/juno node/src/test/java/cab/ml/juno/node/{GgufReaderTest,PhiQuantizedMatVecTest}.java"}

    # f16ToF32 exact values: assertThat(GgufReader.f16ToF32((short) 0x3400)).isEqualTo(0.25f);
    f16 = re.findall(r"f16ToF32\(\(short\)\s*0x([0-9A-Fa-f]+)\)\)\.isEqualTo\((-?[\d.]+)f\)", src)
    out["f16_exact"] = [[int(h, 16), float(v)] for h, v in f16]
    assert len(out["f16_exact"]) == 4

    # Q6_K golden block
    at = src.index("q6k_single_block_golden_values")
    ql, p = java_bytes(src, "ql", at)
    qh, p = java_bytes(src, "qh", p)
    sc, p = java_bytes(src, "sc", p)
    assert (len(ql), len(qh), len(sc)) == (128, 64, 16)
    d16 = int(re.compile(r"short d_f16 = 0x([0-9A-Fa-f]+)").search(src, p).group(1), 16)
    end = src.index("q6k_output_range_bounded")
    exp = re.findall(r"actual\[(\d+)\]\)\.isCloseTo\((-?[\d.]+)f", src[p:end])
    eps = float(re.search(r"float eps = ([\d.]+)f", src[p:end]).group(1))
    block = ql + qh + sc + [d16 & 0xFF, d16 >> 8]
    assert len(block) == 210 and len(exp) == 14
    out["q6k_golden"] = {"block": block, "expected": [[int(i), float(v)] for i, v in exp], "eps": eps}

    # Q6_K range block: ql/qh all 0xFF, sc all 1, d = 1.0 -> |v| <= 32
    out["q6k_range"] = {"block": [0xFF] * 192 + [1] * 16 + [0x00, 0x3C], "abs_max": 32.0}

    # Q4_K all-zero quants, d=1.0 dmin=0 -> exact zeros
    out["q4k_all_zero"] = {"block": [0x00, 0x3C, 0x00, 0x00] + [0] * 12 + [0] * 128, "expected_all": 0.0}
    # Q4_K nibble split: qs[0]=0xF0, sc[0]=1, d=1.0, dmin=0 -> out[0] == 0, size 256
    blk = [0x00, 0x3C, 0x00, 0x00] + [1] + [0] * 11 + [0xF0] + [0] * 127
    out["q4k_nibble_split"] = {"block": blk, "expected": [[0, 0.0]], "size": 256}

    # Q8_0: scale 0.5 (0x3800), values 0..31 -> 0.5*i within 1e-3
    out["q8_0_half_i"] = {"block": [0x00, 0x38] + list(range(32)), "expected": [0.5 * i for i in range(32)],
                          "eps": 1e-3}

    # PhiQuantizedMatVecTest: quantised matvec == dequantise-then-matvec within 1e-3, x = ones
    one = [0x00, 0x3C, 0x00, 0x00] + [1] + [0] * 11 + [0xFF] * 128
    out["q4k_one_block_dot"] = {"block": one, "cols": 256, "x": "ones", "eps": 1e-3}

    def fill(scale, qs):  # fillQ4KBlock
        f16s = [0x3C00, 0x4000, 0x4200, 0x4400]
        d = f16s[min(scale - 1, 3)]
        return [d & 0xFF, d >> 8, 0, 0] + [1] + [0] * 11 + [qs] * 128

    out["q4k_three_rows"] = {"blocks": fill(1, 0x11) + fill(2, 0x22) + fill(3, 0x33), "rows": 3, "cols": 256,
                             "x": "ones", "eps": 1e-3}
    out["q6k_golden_dot"] = {"block": block, "cols": 256, "x": "ones", "eps": 1e-3}
    # raw byte counts (PhiQuantizedMatVecTest :170-190, GgufReader.rawByteCount :347-360)
    out["raw_bytes"] = [{"type": 12, "nelems": 256 * 32, "bytes": 32 * 144}]

    # cross-check the Phi test carries the same golden Q6_K block
    phi = open(os.path.join(node_test, "PhiQuantizedMatVecTest.java"), encoding="utf-8").read()
    at = phi.index("q6k_quantizedTensor_matchesDequantMatVec")
    ql2, p = java_bytes(phi, "ql", at)
    qh2, p = java_bytes(phi, "qh", p)
    sc2, p = java_bytes(phi, "sc", p)
    assert ql2 + qh2 + sc2 == ql + qh + sc

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_known_answers.json")
    with open(dst, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", dst)


if __name__ == "__main__":
    main(sys.argv[1])
