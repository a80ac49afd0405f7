// TEST INFRASTRUCTURE ONLY.
//
// Just enough of HLSL's vector types and intrinsics, written in C++, for the reference's block
// compression shaders (src/shaders/BlockCompressCommon.hlsli, CompressBC1-5.hlsl) to compile and run
// on the CPU.  Every operation is a single binary32 operation evaluated in source order (the
// translation units are built with -ffp-contract=off), components first to last; round() rounds
// halves to even, min / max return the other operand when one is a NaN, as the HLSL intrinsics do.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstring>

typedef uint32_t uint;

// HLSL's vector<T, N>; vec2 / vec3 / vec4 are its aliases (so a function template over
// vector<int, C> accepts an int3).
template <typename T, int N>
struct vector;
template <typename T>
using vec1 = vector<T, 1>;
template <typename T>
using vec2 = vector<T, 2>;
template <typename T>
using vec3 = vector<T, 3>;
template <typename T>
using vec4 = vector<T, 4>;

// One component: converts to and from its scalar, so scalar arithmetic applies to it.
template <typename T>
struct vector<T, 1>
{
    T x;
    vector() : x(T()) {}
    vector(T s) : x(s) {}
    template <typename U>
    explicit vector(const vector<U, 1>& o) : x(T(o.x)) {}
    operator T() const { return x; }
    T& operator[](int) { return x; }
    const T& operator[](int) const { return x; }
};

template <typename T>
struct vector<T, 2>
{
    union
    {
        struct { T x, y; };
        struct { T r, g; };
    };
    vector() : x(T()), y(T()) {}
    vector(T s) : x(s), y(s) {}
    vector(T a, T b) : x(a), y(b) {}
    template <typename U>
    explicit vector(const vector<U, 2>& o) : x(T(o.x)), y(T(o.y)) {}
    T& operator[](int i) { return (&x)[i]; }
    const T& operator[](int i) const { return (&x)[i]; }
};

template <typename T>
struct vector<T, 3>
{
    union
    {
        struct { T x, y, z; };
        struct { T r, g, b; };
    };
    vector() : x(T()), y(T()), z(T()) {}
    vector(T s) : x(s), y(s), z(s) {}
    vector(T a, T b_, T c) : x(a), y(b_), z(c) {}
    template <typename U>
    explicit vector(const vector<U, 3>& o) : x(T(o.x)), y(T(o.y)), z(T(o.z)) {}
    T& operator[](int i) { return (&x)[i]; }
    const T& operator[](int i) const { return (&x)[i]; }
};

// The first three components of a four-component vector, as HLSL's .rgb swizzle: reads as a vec3,
// assigns component-wise.
template <typename T>
struct swizzle3
{
    T a, b, c;
    operator vec3<T>() const { return vec3<T>(a, b, c); }
    swizzle3& operator=(const vec3<T>& v)
    {
        a = v.x;
        b = v.y;
        c = v.z;
        return *this;
    }
};

template <typename T>
struct vector<T, 4>
{
    union
    {
        struct { T x, y, z, w; };
        struct { T r, g, b, a; };
        swizzle3<T> rgb;
        swizzle3<T> xyz;
    };
    vector() : x(T()), y(T()), z(T()), w(T()) {}
    vector(T s) : x(s), y(s), z(s), w(s) {}
    vector(T a_, T b_, T c, T d) : x(a_), y(b_), z(c), w(d) {}
    vector(const vec3<T>& v, T d) : x(v.x), y(v.y), z(v.z), w(d) {}
    vector(const vec2<T>& u, const vec2<T>& v) : x(u.x), y(u.y), z(v.x), w(v.y) {}
    vector(const vector& o) : x(o.x), y(o.y), z(o.z), w(o.w) {}
    template <typename U>
    explicit vector(const vector<U, 4>& o) : x(T(o.x)), y(T(o.y)), z(T(o.z)), w(T(o.w)) {}
    vector& operator=(const vector& o)
    {
        x = o.x;
        y = o.y;
        z = o.z;
        w = o.w;
        return *this;
    }
    T& operator[](int i) { return (&x)[i]; }
    const T& operator[](int i) const { return (&x)[i]; }
    // a four-component swizzle such as .agbr, spelled by the transform as .swizzle4(3, 1, 2, 0)
    vector swizzle4(int i0, int i1, int i2, int i3) const { return vector((&x)[i0], (&x)[i1], (&x)[i2], (&x)[i3]); }
};

typedef vec2<float> float2;
typedef vec3<float> float3;
typedef vec4<float> float4;
typedef vec2<int> int2;
typedef vec3<int> int3;
typedef vec4<int> int4;
typedef vec2<uint> uint2;
typedef vec3<uint> uint3;
typedef vec4<uint> uint4;
typedef vec3<bool> bool3;
typedef vec4<bool> bool4;

// ---- component-wise arithmetic ----------------------------------------------------------------
#define HLSL_BINARY(op)                                                                                          \
    template <typename T>                                                                                         \
    vec2<T> operator op(const vec2<T>& a, const vec2<T>& b) { return vec2<T>(a.x op b.x, a.y op b.y); }          \
    template <typename T>                                                                                         \
    vec3<T> operator op(const vec3<T>& a, const vec3<T>& b) { return vec3<T>(a.x op b.x, a.y op b.y, a.z op b.z); } \
    template <typename T>                                                                                         \
    vec4<T> operator op(const vec4<T>& a, const vec4<T>& b)                                                      \
    {                                                                                                             \
        return vec4<T>(a.x op b.x, a.y op b.y, a.z op b.z, a.w op b.w);                                           \
    }                                                                                                             \
    template <typename T>                                                                                         \
    vec3<T> operator op(const swizzle3<T>& a, const vec3<T>& b) { return vec3<T>(a) op b; }                      \
    template <typename T>                                                                                         \
    vec3<T> operator op(const vec3<T>& a, const swizzle3<T>& b) { return a op vec3<T>(b); }                      \
    template <typename T>                                                                                         \
    vec3<T> operator op(const swizzle3<T>& a, const swizzle3<T>& b) { return vec3<T>(a) op vec3<T>(b); }
HLSL_BINARY(+)
HLSL_BINARY(-)
HLSL_BINARY(*)
HLSL_BINARY(/)
#undef HLSL_BINARY

// vector (op) scalar and scalar (op) vector: the scalar is converted to the component type first
#define HLSL_SCALAR(op)                                                                                  \
    inline float3 operator op(const float3& a, float s) { return a op float3(s); }                        \
    inline float3 operator op(float s, const float3& a) { return float3(s) op a; }                        \
    inline float3 operator op(const swizzle3<float>& a, float s) { return float3(a) op float3(s); }       \
    inline float3 operator op(float s, const swizzle3<float>& a) { return float3(s) op float3(a); }       \
    inline float4 operator op(const float4& a, float s) { return a op float4(s); }                        \
    inline float4 operator op(float s, const float4& a) { return float4(s) op a; }                        \
    inline float2 operator op(const float2& a, float s) { return a op float2(s); }                        \
    inline float2 operator op(float s, const float2& a) { return float2(s) op a; }                        \
    inline uint2 operator op(const uint2& a, uint s) { return a op uint2(s); }                            \
    inline uint2 operator op(const uint2& a, int s) { return a op uint2(uint(s)); }
HLSL_SCALAR(+)
HLSL_SCALAR(-)
HLSL_SCALAR(*)
HLSL_SCALAR(/)
#undef HLSL_SCALAR
inline float3 operator/(const float3& a, int s) { return a / float3(float(s)); }

template <typename V, typename W>
V& operator+=(V& a, const W& b) { a = a + b; return a; }
template <typename V, typename W>
V& operator-=(V& a, const W& b) { a = a - b; return a; }
template <typename V, typename W>
V& operator*=(V& a, const W& b) { a = a * b; return a; }
template <typename V, typename W>
V& operator/=(V& a, const W& b) { a = a / b; return a; }

inline bool3 operator==(const float3& a, float s) { return bool3(a.x == s, a.y == s, a.z == s); }
inline bool3 operator==(const float3& a, double s) { return a == float(s); }

// ---- intrinsics ---------------------------------------------------------------------------------
inline float hlsl_min(float a, float b) { return std::fmin(a, b); }
inline float hlsl_max(float a, float b) { return std::fmax(a, b); }
inline float min(float a, float b) { return hlsl_min(a, b); }
inline float max(float a, float b) { return hlsl_max(a, b); }
inline int min(int a, int b) { return a < b ? a : b; }
inline int max(int a, int b) { return a > b ? a : b; }
inline uint min(uint a, uint b) { return a < b ? a : b; }
inline uint max(uint a, uint b) { return a > b ? a : b; }
inline float3 min(const float3& a, const float3& b) { return float3(min(a.x, b.x), min(a.y, b.y), min(a.z, b.z)); }
inline float3 max(const float3& a, const float3& b) { return float3(max(a.x, b.x), max(a.y, b.y), max(a.z, b.z)); }
inline float saturate(float v) { return hlsl_min(hlsl_max(v, 0.f), 1.f); } // NaN -> 0, as the DXIL saturate
inline float3 saturate(const float3& v) { return float3(saturate(v.x), saturate(v.y), saturate(v.z)); }
inline float clamp(float v, float lo, float hi) { return hlsl_min(hlsl_max(v, lo), hi); }
inline int clamp(int v, int lo, int hi) { return min(max(v, lo), hi); }
inline uint clamp(uint v, uint lo, uint hi) { return min(max(v, lo), hi); }
inline float round(float v) { return std::nearbyintf(v); } // halves to even (the default rounding mode)
inline float3 round(const float3& v) { return float3(round(v.x), round(v.y), round(v.z)); }
inline float abs(float v) { return std::fabs(v); }
inline float dot(const float3& a, const float3& b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
inline float dot(const float4& a, const float4& b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
inline float lerp(float a, float b, float t) { return a + t * (b - a); }
inline float3 lerp(const float3& a, const float3& b, float t) { return a + t * (b - a); }
inline bool3 hlsl_or(const bool3& a, const bool3& b) { return bool3(a.x || b.x, a.y || b.y, a.z || b.z); }
inline float3 select(const bool3& c, const float3& a, const float3& b)
{
    return float3(c.x ? a.x : b.x, c.y ? a.y : b.y, c.z ? a.z : b.z);
}

// ---- more of the same, for the BC7 encoder (src/shaders/CompressBC7.hlsl) ------------------------------
inline float4 min(const float4& a, const float4& b) { return float4(min(a.x, b.x), min(a.y, b.y), min(a.z, b.z), min(a.w, b.w)); }
inline float4 max(const float4& a, const float4& b) { return float4(max(a.x, b.x), max(a.y, b.y), max(a.z, b.z), max(a.w, b.w)); }
inline float4 saturate(const float4& v) { return float4(saturate(v.x), saturate(v.y), saturate(v.z), saturate(v.w)); }
inline float dot(float a, float b) { return a * b; }
inline bool4 operator==(const float4& a, float s) { return bool4(a.x == s, a.y == s, a.z == s, a.w == s); }
inline bool hlsl_or(bool a, bool b) { return a || b; }
inline bool4 hlsl_or(const bool4& a, const bool4& b) { return bool4(a.x || b.x, a.y || b.y, a.z || b.z, a.w || b.w); }
inline float select(bool c, float a, float b) { return c ? a : b; }
inline float4 select(const bool4& c, const float4& a, const float4& b)
{
    return float4(c.x ? a.x : b.x, c.y ? a.y : b.y, c.z ? a.z : b.z, c.w ? a.w : b.w);
}
inline float3 operator/(const float3& a, uint s) { return a / float3(float(s)); }
inline float4 operator/(const float4& a, uint s) { return a / float4(float(s)); }
inline uint countbits(uint v) { return uint(__builtin_popcount(v)); }

// integer vectors with an integer scalar
#define HLSL_INT_SCALAR(op)                                                                          \
    inline int3 operator op(const int3& a, int s) { return int3(a.x op s, a.y op s, a.z op s); }      \
    inline int4 operator op(const int4& a, int s) { return int4(a.x op s, a.y op s, a.z op s, a.w op s); }
HLSL_INT_SCALAR(+)
HLSL_INT_SCALAR(*)
HLSL_INT_SCALAR(>>)
HLSL_INT_SCALAR(&)
HLSL_INT_SCALAR(|)
#undef HLSL_INT_SCALAR

// Thread-group machinery of the BC7 shader's single-mode path, for ONE thread running alone: the
// harness clears the group-shared counters before every call, so the thread is the only one of its
// group and of its wave, and the re-ordering hands it back its own block.
#define groupshared static
inline void InterlockedAdd(uint& target, uint value, uint& original)
{
    original = target;
    target += value;
}
inline uint WaveActiveCountBits(bool) { return 1; }
inline bool WaveIsFirstLane() { return true; }
inline uint WaveReadLaneFirst(uint v) { return v; }
inline uint WavePrefixCountBits(bool) { return 0; }
inline void GroupMemoryBarrierWithGroupSync() {}

// a scalar array seen as an array of one-component vectors (same storage)
template <typename T>
inline const vector<T, 1>* hlsl_as_vec1(const T* p) { return reinterpret_cast<const vector<T, 1>*>(p); }

// ---- resources ------------------------------------------------------------------------------------
// A read-only four-component texture: texels outside the image read as zero in every component.
template <typename T>
struct Texture2D
{
    const T* data = nullptr;
    int width = 0, height = 0;
    T operator[](const uint2& p) const
    {
        if (p.x >= uint(width) || p.y >= uint(height))
            return T(0.f);
        return data[size_t(p.y) * width + p.x];
    }
};

template <typename T>
struct RWTexture2D
{
    T* data = nullptr;
    int width = 0, height = 0;
    T scratch;
    T& operator[](const uint2& p)
    {
        if (p.x >= uint(width) || p.y >= uint(height))
            return scratch;
        return data[size_t(p.y) * width + p.x];
    }
};

struct ByteAddressBuffer
{
    const uint32_t* data = nullptr;
    uint Load(uint byteOffset) const { return data[byteOffset / 4]; }
};

// binding helpers of the shaders: a declaration is just a global here
#define NTC_DECLARE_CBUFFER(decl, reg, space) decl
#define NTC_DECLARE_SAMPLER(decl, reg, space) decl
#define NTC_DECLARE_SRV(decl, reg, space) decl
#define NTC_DECLARE_UAV(decl, reg, space) decl
