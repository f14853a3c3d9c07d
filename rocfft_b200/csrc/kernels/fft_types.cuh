// Complex value types and small arithmetic helpers shared by every kernel and
// by the generated butterflies.  Compiles as plain C++ too (the host-side
// butterfly check builds the generated header with g++), hence the fallbacks.
#pragma once
#if defined(__CUDACC__)
#include <cuda_runtime.h>
#define B200FFT_DEVICE __device__ __forceinline__
#else
struct float2
{
    float x, y;
};
struct double2
{
    double x, y;
};
#define B200FFT_DEVICE inline
#endif

namespace b200fft
{
    template <typename T>
    struct cx;
    template <>
    struct cx<float>
    {
        using type = float2;
    };
    template <>
    struct cx<double>
    {
        using type = double2;
    };

    template <typename T2>
    B200FFT_DEVICE T2 cmul(const T2 a, const T2 b)
    {
        T2 r;
        r.x = a.x * b.x - a.y * b.y;
        r.y = a.x * b.y + a.y * b.x;
        return r;
    }
    // a * conj(b)
    template <typename T2>
    B200FFT_DEVICE T2 cmulc(const T2 a, const T2 b)
    {
        T2 r;
        r.x = a.x * b.x + a.y * b.y;
        r.y = a.y * b.x - a.x * b.y;
        return r;
    }
    template <typename T2>
    B200FFT_DEVICE T2 cswap(const T2 a)
    {
        T2 r;
        r.x = a.y;
        r.y = a.x;
        return r;
    }

    // forward DFT of W points held in registers, natural order in and out;
    // specialisations come from the generated header
    template <int W, typename T2>
    struct Butterfly;

    template <typename T2>
    struct Butterfly<1, T2>
    {
        static B200FFT_DEVICE void run(T2 (&)[1]) {}
    };
} // namespace b200fft
