#!/usr/bin/env python
"""TEST INFRASTRUCTURE ONLY.

Makes the copies of the reference's src/TextureSet.h and src/TextureSet.cpp from which
`oracle/build_ref.sh --with-ntcb` builds oracle/_ref/libntc_ref_ntcb.so: LibNTC with its CUDA
decompression routed through libntcb200.so, everything else unmodified.  Nothing of the reference
is stored in this repository: the copies are written under oracle/_ref/ (git-ignored) and the three
edits are anchored on the two declarations they attach to.

    patch_texture_set.py <reference-source-dir> <output-dir>

Edits:
  1. TextureSet.h: the member function DecompressThroughNtcb is declared beside Decompress (a
     non-virtual member function: the layout of the class, which the unmodified translation units
     also see, does not change).
  2. TextureSet.cpp: TextureSet::Decompress hands a set that was loaded from a file and has no
     reference image (the only case a decoder-only client meets) to that function.
  3. TextureSet.cpp: oracle/texture_set_ntcb.inl, which defines it, is included at the end.
"""
import os
import sys

DECLARATION = "Status Decompress(DecompressionStats* pOutStats, bool useInt8Weights) override;"
DEFINITION = "Status TextureSet::Decompress(DecompressionStats* pOutStats, bool useInt8Weights)\n{\n"


def main() -> int:
    reference, out = sys.argv[1], sys.argv[2]
    here = os.path.dirname(os.path.abspath(__file__))
    os.makedirs(out, exist_ok=True)

    with open(os.path.join(reference, "src", "TextureSet.h")) as f:
        header = f.read()
    if header.count(DECLARATION) != 1:
        print("patch_texture_set.py: the declaration of TextureSet::Decompress was not found", file=sys.stderr)
        return 1
    header = header.replace(
        DECLARATION, DECLARATION + "\n\n    Status DecompressThroughNtcb(DecompressionStats* pOutStats, bool useInt8Weights);")
    with open(os.path.join(out, "TextureSet.h"), "w") as f:
        f.write(header)

    with open(os.path.join(reference, "src", "TextureSet.cpp")) as f:
        source = f.read()
    if source.count(DEFINITION) != 1:
        print("patch_texture_set.py: the definition of TextureSet::Decompress was not found", file=sys.stderr)
        return 1
    route = ("    if (m_networkState == TextureSetNetworkState::Complete && GetValidChannelMask() == 0)\n"
             "        return DecompressThroughNtcb(pOutStats, useInt8Weights);\n\n")
    source = source.replace(DEFINITION, DEFINITION + route)
    source += '\n#include "%s"\n' % os.path.join(here, "texture_set_ntcb.inl")
    with open(os.path.join(out, "TextureSet.cpp"), "w") as f:
        f.write(source)
    return 0


if __name__ == "__main__":
    sys.exit(main())
