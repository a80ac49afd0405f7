#!/usr/bin/env python
"""TEST INFRASTRUCTURE ONLY.

Turns the reference's block-compression shader sources into text a C++ compiler accepts, without
changing what they compute:
  * `inout T name` / `out T name` parameters become `T& name` (array parameters, which C++ already
    passes by address, only lose the keyword);
  * floating literals without a suffix get an `f`: in HLSL an unsuffixed literal takes the type of the
    expression it appears in (binary32 here), in C++ it would turn the whole expression into binary64;
  * loop attributes ([unroll], [loop], ...) and the entry point's [numthreads] / semantics go;
  * the boolean intrinsic `or(` becomes hlsl_or( (`or` is an operator keyword in C++);
  * four-component swizzles (`.agbr`) become `.swizzle4(3, 1, 2, 0)`, and a scalar array passed where
    the callee is instantiated for one-component vectors (`<1>(alphaPixels`) is passed as such;
  * the constant buffer, declared `static const` for C++ in the source, becomes an ordinary global
    that the harness fills in.
Nothing of the output is stored in the repository: it is written under oracle/_ref/.

    transform_hlsl.py <input.hlsl> <output.h> [entry-point-name]
"""
import re
import sys


def transform(text: str, entry: str) -> str:
    text = re.sub(r"\[(unroll|loop|branch|flatten)(\([^\]]*\))?\]", "", text)
    text = re.sub(r"\[numthreads\([^\]]*\)\]", "", text)
    text = re.sub(r"\s*:\s*SV_\w+", "", text)
    # out / inout parameters: arrays keep their form, everything else becomes a reference
    text = re.sub(r"\b(?:inout|out)\s+(\w+)\s+(\w+)\s*\[", r"\1 \2[", text)
    text = re.sub(r"\b(?:inout|out)\s+(\w+)\s+(\w+)", r"\1& \2", text)
    # unsuffixed floating literals -> binary32 (not inside identifiers or hexadecimal numbers)
    text = re.sub(r"(?<![\w.])(\d+\.\d*(?:[eE][+-]?\d+)?|\.\d+(?:[eE][+-]?\d+)?|\d+[eE][+-]?\d+)(?![\w.])", r"\1f", text)
    text = re.sub(r"\bor\(", "hlsl_or(", text)
    text = re.sub(r"\.([rgba]{4})\b", lambda m: ".swizzle4(%s)" % ", ".join(str("rgba".index(ch)) for ch in m.group(1)), text)
    text = re.sub(r"<1>\((\w+Pixels)\b", r"<1>(hlsl_as_vec1(\1)", text)
    text = text.replace("static const NtcBlockCompressConstants g_Const;", "NtcBlockCompressConstants g_Const;")
    text = re.sub(r"\bvoid\s+main\s*\(", "void %s(" % entry, text)
    return text


if __name__ == "__main__":
    source, target = sys.argv[1], sys.argv[2]
    entry = sys.argv[3] if len(sys.argv) > 3 else "main"
    with open(source) as f:
        result = transform(f.read(), entry)
    with open(target, "w") as f:
        f.write(result)
