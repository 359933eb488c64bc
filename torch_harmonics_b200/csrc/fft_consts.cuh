// Generated constants: cos / sin of 2 pi k / R for the composite in-register butterflies (evaluated in double, rounded to float).
#pragma once
namespace shtb200 {
template <int R> struct RootTab;
template <> struct RootTab<6> {
    static __host__ __device__ constexpr float c(int k) { constexpr float t[6] = {1.0f, 0.5f, -0.5f, -1.0f, -0.5f, 0.5f}; return t[k]; }
    static __host__ __device__ constexpr float s(int k) { constexpr float t[6] = {0.0f, 0.8660254037844386f, 0.8660254037844387f, 0.0f, -0.8660254037844384f, -0.8660254037844386f}; return t[k]; }
};
template <> struct RootTab<8> {
    static __host__ __device__ constexpr float c(int k) { constexpr float t[8] = {1.0f, 0.7071067811865476f, 0.0f, -0.7071067811865475f, -1.0f, -0.7071067811865477f, 0.0f, 0.7071067811865474f}; return t[k]; }
    static __host__ __device__ constexpr float s(int k) { constexpr float t[8] = {0.0f, 0.7071067811865475f, 1.0f, 0.7071067811865476f, 0.0f, -0.7071067811865475f, -1.0f, -0.7071067811865477f}; return t[k]; }
};
template <> struct RootTab<9> {
    static __host__ __device__ constexpr float c(int k) { constexpr float t[9] = {1.0f, 0.766044443118978f, 0.17364817766693041f, -0.5f, -0.9396926207859083f, -0.9396926207859084f, -0.5f, 0.17364817766692997f, 0.7660444431189778f}; return t[k]; }
    static __host__ __device__ constexpr float s(int k) { constexpr float t[9] = {0.0f, 0.6427876096865393f, 0.984807753012208f, 0.8660254037844387f, 0.3420201433256689f, -0.34202014332566866f, -0.8660254037844384f, -0.9848077530122081f, -0.6427876096865396f}; return t[k]; }
};
template <> struct RootTab<10> {
    static __host__ __device__ constexpr float c(int k) { constexpr float t[10] = {1.0f, 0.8090169943749475f, 0.30901699437494745f, -0.30901699437494734f, -0.8090169943749473f, -1.0f, -0.8090169943749476f, -0.30901699437494756f, 0.30901699437494723f, 0.8090169943749473f}; return t[k]; }
    static __host__ __device__ constexpr float s(int k) { constexpr float t[10] = {0.0f, 0.5877852522924731f, 0.9510565162951535f, 0.9510565162951536f, 0.5877852522924732f, 0.0f, -0.587785252292473f, -0.9510565162951535f, -0.9510565162951536f, -0.5877852522924734f}; return t[k]; }
};
template <> struct RootTab<12> {
    static __host__ __device__ constexpr float c(int k) { constexpr float t[12] = {1.0f, 0.8660254037844387f, 0.5f, 0.0f, -0.5f, -0.8660254037844387f, -1.0f, -0.8660254037844388f, -0.5f, 0.0f, 0.5f, 0.8660254037844384f}; return t[k]; }
    static __host__ __device__ constexpr float s(int k) { constexpr float t[12] = {0.0f, 0.5f, 0.8660254037844386f, 1.0f, 0.8660254037844387f, 0.5f, 0.0f, -0.5f, -0.8660254037844384f, -1.0f, -0.8660254037844386f, -0.5f}; return t[k]; }
};
template <> struct RootTab<15> {
    static __host__ __device__ constexpr float c(int k) { constexpr float t[15] = {1.0f, 0.9135454576426009f, 0.6691306063588582f, 0.30901699437494745f, -0.10452846326765333f, -0.5f, -0.8090169943749473f, -0.9781476007338057f, -0.9781476007338057f, -0.8090169943749476f, -0.5f, -0.10452846326765423f, 0.30901699437494723f, 0.6691306063588585f, 0.913545457642601f}; return t[k]; }
    static __host__ __device__ constexpr float s(int k) { constexpr float t[15] = {0.0f, 0.40673664307580015f, 0.7431448254773941f, 0.9510565162951535f, 0.9945218953682734f, 0.8660254037844387f, 0.5877852522924732f, 0.20791169081775931f, -0.20791169081775907f, -0.587785252292473f, -0.8660254037844384f, -0.9945218953682733f, -0.9510565162951536f, -0.743144825477394f, -0.40673664307580015f}; return t[k]; }
};
template <> struct RootTab<16> {
    static __host__ __device__ constexpr float c(int k) { constexpr float t[16] = {1.0f, 0.9238795325112867f, 0.7071067811865476f, 0.38268343236508984f, 0.0f, -0.3826834323650897f, -0.7071067811865475f, -0.9238795325112867f, -1.0f, -0.9238795325112868f, -0.7071067811865477f, -0.38268343236509034f, 0.0f, 0.38268343236509f, 0.7071067811865474f, 0.9238795325112865f}; return t[k]; }
    static __host__ __device__ constexpr float s(int k) { constexpr float t[16] = {0.0f, 0.3826834323650898f, 0.7071067811865475f, 0.9238795325112867f, 1.0f, 0.9238795325112867f, 0.7071067811865476f, 0.3826834323650899f, 0.0f, -0.38268343236508967f, -0.7071067811865475f, -0.9238795325112865f, -1.0f, -0.9238795325112866f, -0.7071067811865477f, -0.3826834323650904f}; return t[k]; }
};
}  // namespace shtb200
