#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.
#
# Builds the UNMODIFIED reference library (LibNTC) from its own sources, where they lie, into
# oracle/_ref/libntc_ref.so together with the plain-C drivers oracle/ref_harness.cpp and
# oracle/ref_harness_producers.cu.  The result is
# the parity checker and the benchmark's reference arm; it is never linked into the product.
#
# The reference's own CMake build needs network access (FetchContent) and the libdeflate submodule,
# so the sources are compiled directly with the same definitions and nvcc flags its CMake files set
# (src/CMakeLists.txt:15-44,120-135): C++17, --expt-relaxed-constexpr --extended-lambda
# --use_fast_math, separable compilation, CUDA only (no DX12 / Vulkan / prebuilt shaders).
# Differences from the stock build, none of which touches the decode path:
#   * target architecture sm_100 instead of the default 75/86/89 list;
#   * src/GDeflate.cpp is replaced by oracle/gdeflate_stub.cpp (libdeflate sources are absent);
#   * src/Shaders.cpp is left out, exactly as the stock build does without prebuilt shaders.
#
# With --with-ntcb a second library, oracle/_ref/libntc_ref_ntcb.so, is built from the same objects
# except TextureSet.cpp, which is compiled from a patched copy (oracle/patch_texture_set.py +
# oracle/texture_set_ntcb.inl) whose Decompress calls libntcb200.so: the reference's public API
# (ntc::CreateContext, IContext, ITextureSet) with this repository's decoder behind it.  It proves the
# integration described in INTEGRATION.md and is test infrastructure like the rest of oracle/.
#
# Usage: oracle/build_ref.sh [--with-ntcb] [reference-source-dir]
#   (default: $NTC_REFERENCE_DIR, else a checkout named `reference` beside this repository)
set -euo pipefail

HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
WITH_NTCB=0
if [ "${1:-}" = "--with-ntcb" ]; then
    WITH_NTCB=1
    shift
fi
REF="${1:-${NTC_REFERENCE_DIR:-$HERE/../../reference}}"
OUT="$HERE/_ref"
OBJ="$OUT/obj"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
CXX="${CXX:-g++}"
JOBS="${JOBS:-$(nproc)}"

if [ ! -f "$REF/src/Inference.cu" ]; then
    echo "build_ref.sh: reference sources not found under $REF" >&2
    exit 3
fi

mkdir -p "$OBJ"

# The reference generates VersionInfo.h from src/VersionInfoTemplate.h at configure time.
cat > "$OBJ/VersionInfo.h" <<'EOF'
#define NTC_VERSION_MAJOR 0
#define NTC_VERSION_MINOR 9
#define NTC_VERSION_POINT 2
#define NTC_VERSION_BRANCH "reference"
#define NTC_VERSION_HASH "unmodified"
#define NTC_VERSION_FULL "0.9.2 reference-unmodified"
EOF

DEFS="-DNTC_WITH_CUDA=1 -DNTC_WITH_VULKAN=0 -DNTC_WITH_DX12=0 -DNTC_WITH_PREBUILT_SHADERS=0 \
-DNTC_STATIC=1 -DNTC_CUDA_MIN_COMPUTE_MAJOR=7 -DNTC_CUDA_MIN_COMPUTE_MINOR=5"
INCS="-I$OBJ -I$REF/include -I$REF/src -I$REF/external/rapidjson/include -I/usr/local/cuda/include"

CU_SOURCES="Inference Quantizer Regression RegressionFast RegressionStable Optimizer ImageProcessing CudaRandomGen"
CPP_SOURCES="AdaptiveCompressionSession BinaryChunkBuilder Context CoopVecWeightConverter CudaDeviceGuard \
Errors FeatureGridHost FeatureGridMath GraphicsResources JsonFileFormat JsonSerialization PublicFunctions \
SharedTexture Stream TextureMetadata TextureSet TextureSetMetadata ThreadPool WeightLayout"

compile_cu() {
    "$NVCC" -arch=sm_100 -std=c++17 -O3 --expt-relaxed-constexpr --extended-lambda --use_fast_math \
        -rdc=true -Xcompiler -fPIC -Xcompiler -fno-strict-aliasing $DEFS $INCS \
        -c "$REF/src/$1.cu" -o "$OBJ/$1.cu.o"
}
compile_harness_cu() {
    "$NVCC" -arch=sm_100 -std=c++17 -O3 --expt-relaxed-constexpr --extended-lambda --use_fast_math \
        -rdc=true -Xcompiler -fPIC -Xcompiler -fno-strict-aliasing $DEFS $INCS \
        -c "$HERE/$1.cu" -o "$OBJ/$1.cu.o"
}
compile_cpp() {
    "$CXX" -std=c++17 -O2 -fPIC -fno-strict-aliasing $DEFS $INCS -c "$2" -o "$OBJ/$1.o"
}
export -f compile_cu compile_harness_cu compile_cpp
export NVCC CXX DEFS INCS OBJ REF HERE

{
    for s in $CU_SOURCES; do echo "compile_cu $s"; done
    for s in $CPP_SOURCES; do echo "compile_cpp $s $REF/src/$s.cpp"; done
    echo "compile_cpp gdeflate_stub $HERE/gdeflate_stub.cpp"
    echo "compile_cpp ref_harness $HERE/ref_harness.cpp"
    echo "compile_harness_cu ref_harness_producers"
} | xargs -P "$JOBS" -I{} bash -c '{}'

OBJECTS=""
for s in $CU_SOURCES; do OBJECTS="$OBJECTS $OBJ/$s.cu.o"; done
for s in $CPP_SOURCES gdeflate_stub ref_harness; do OBJECTS="$OBJECTS $OBJ/$s.o"; done
OBJECTS="$OBJECTS $OBJ/ref_harness_producers.cu.o"

"$NVCC" -arch=sm_100 -shared -o "$OUT/libntc_ref.so" $OBJECTS -lcudart_static -lpthread -ldl -lrt
echo "built $OUT/libntc_ref.so"

# The reference's BC1 - BC5 and BC7 encoders (compute shaders) as C++ on the CPU: src/shaders/CompressBC1-5.hlsl,
# CompressBC7.hlsl and BlockCompressCommon.hlsli, passed through oracle/transform_hlsl.py (parameter qualifiers,
# literal suffixes, attributes, swizzle spelling - nothing that changes the arithmetic) and compiled against
# oracle/hlsl_shim.h without contraction, one translation unit per format (oracle/ref_bc_harness.cpp); BC7 twice,
# with and without its mode buffer, as the reference builds that shader twice.  No graphics API.
BCGEN="$OUT/bc_gen"
mkdir -p "$BCGEN"
python3 "$HERE/transform_hlsl.py" "$REF/src/shaders/BlockCompressCommon.hlsli" "$BCGEN/BlockCompressCommon.hlsli"
: > "$BCGEN/BindingHelpers.hlsli"   # the binding macros come from the shim
BC_FLAGS="-std=c++17 -O2 -fPIC -ffp-contract=off -fno-fast-math -fno-strict-aliasing -w"
BC_OBJECTS=""
for n in 1 2 3 4 5 7; do
    python3 "$HERE/transform_hlsl.py" "$REF/src/shaders/CompressBC$n.hlsl" "$BCGEN/CompressBC$n.hlsl" shader_main
    if [ $n = 7 ]; then
        for modes in 0 1; do
            "$CXX" $BC_FLAGS -I"$HERE" -I"$BCGEN" -I"$REF/include" -DNTC_BC_SHADER="\"CompressBC$n.hlsl\"" -DNTC_BC_FORMAT=$n \
                -DUSE_MODE_BUFFER=$modes -c "$HERE/ref_bc_harness.cpp" -o "$BCGEN/bc${n}_$modes.o"
            BC_OBJECTS="$BC_OBJECTS $BCGEN/bc${n}_$modes.o"
        done
    else
        "$CXX" $BC_FLAGS -I"$HERE" -I"$BCGEN" -I"$REF/include" -DNTC_BC_SHADER="\"CompressBC$n.hlsl\"" -DNTC_BC_FORMAT=$n \
            -c "$HERE/ref_bc_harness.cpp" -o "$BCGEN/bc$n.o"
        BC_OBJECTS="$BC_OBJECTS $BCGEN/bc$n.o"
    fi
done
"$CXX" -shared -o "$OUT/libntc_ref_bc.so" $BC_OBJECTS
echo "built $OUT/libntc_ref_bc.so"

if [ "$WITH_NTCB" = 1 ]; then
    PRODUCT="$HERE/../rtxntc-library_b200"
    if [ ! -f "$PRODUCT/libntcb200.so" ]; then
        echo "build_ref.sh: $PRODUCT/libntcb200.so is not built (make -C rtxntc-library_b200/csrc)" >&2
        exit 4
    fi
    PATCHED="$OUT/obj_ntcb"
    python3 "$HERE/patch_texture_set.py" "$REF" "$PATCHED"
    # the patched copy finds its own TextureSet.h first (same directory), everything else in the reference
    "$CXX" -std=c++17 -O2 -fPIC -fno-strict-aliasing $DEFS -I"$PATCHED" $INCS -I"$HERE/../include" \
        -c "$PATCHED/TextureSet.cpp" -o "$PATCHED/TextureSet.o"
    OBJECTS_NTCB="${OBJECTS/$OBJ\/TextureSet.o/$PATCHED/TextureSet.o}"
    "$NVCC" -arch=sm_100 -shared -o "$OUT/libntc_ref_ntcb.so" $OBJECTS_NTCB -L"$PRODUCT" -lntcb200 \
        -Xlinker -rpath -Xlinker '$ORIGIN/../../rtxntc-library_b200' -lcudart_static -lpthread -ldl -lrt
    echo "built $OUT/libntc_ref_ntcb.so"
fi
