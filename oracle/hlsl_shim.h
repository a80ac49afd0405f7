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

template <typename T>
struct vec2;
template <typename T>
struct vec3;
template <typename T>
struct vec4;

template <typename T>
struct vec2
{
    union
    {
        struct { T x, y; };
        struct { T r, g; };
    };
    vec2() : x(T()), y(T()) {}
    vec2(T s) : x(s), y(s) {}
    vec2(T a, T b) : x(a), y(b) {}
    template <typename U>
    explicit vec2(const vec2<U>& o) : x(T(o.x)), y(T(o.y)) {}
};

template <typename T>
struct vec3
{
    union
    {
        struct { T x, y, z; };
        struct { T r, g, b; };
    };
    vec3() : x(T()), y(T()), z(T()) {}
    vec3(T s) : x(s), y(s), z(s) {}
    vec3(T a, T b_, T c) : x(a), y(b_), z(c) {}
    template <typename U>
    explicit vec3(const vec3<U>& o) : x(T(o.x)), y(T(o.y)), z(T(o.z)) {}
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
struct vec4
{
    union
    {
        struct { T x, y, z, w; };
        struct { T r, g, b, a; };
        swizzle3<T> rgb;
        swizzle3<T> xyz;
    };
    vec4() : x(T()), y(T()), z(T()), w(T()) {}
    vec4(T s) : x(s), y(s), z(s), w(s) {}
    vec4(T a_, T b_, T c, T d) : x(a_), y(b_), z(c), w(d) {}
    vec4(const vec3<T>& v, T d) : x(v.x), y(v.y), z(v.z), w(d) {}
    vec4(const vec2<T>& u, const vec2<T>& v) : x(u.x), y(u.y), z(v.x), w(v.y) {}
    vec4(const vec4& o) : x(o.x), y(o.y), z(o.z), w(o.w) {}
    vec4& operator=(const vec4& o)
    {
        x = o.x;
        y = o.y;
        z = o.z;
        w = o.w;
        return *this;
    }
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
