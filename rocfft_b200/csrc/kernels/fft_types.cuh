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

    // Arithmetic helpers the generated butterflies are written in, so that the same straight-line
    // code serves scalars and the packed pairs below: a * b + c, a * c + b * s, a * c - b * s.
    template <typename T>
    B200FFT_DEVICE T bfma(const T a, const T b, const T c)
    {
        return a * b + c;
    }
    template <typename T>
    B200FFT_DEVICE T madd(const T a, const T c, const T b, const T s)
    {
        return a * c + b * s;
    }
    template <typename T>
    B200FFT_DEVICE T msub(const T a, const T c, const T b, const T s)
    {
        return a * c - b * s;
    }

#if defined(__CUDACC__)
    // Two single-precision values that travel through the packed fp32 instructions of sm_100
    // (add / mul / fma on an aligned register pair: one issue slot for two lanes).  The kernels
    // that use it put the SAME component of TWO independent transforms into one pair — real parts
    // of columns a and b in one pk2, imaginary parts in another — so the generated butterflies run
    // unchanged on `pk2` scalars and every instruction serves two transforms, with no shuffling
    // between the halves of a pair.
    struct pk2
    {
        float2 v;
        pk2() = default;
        __device__ __forceinline__ pk2(float2 a)
            : v(a)
        {
        }
        __device__ __forceinline__ pk2(float a, float b)
            : v(make_float2(a, b))
        {
        }
        // literal constants of the butterflies: the same value in both lanes
        __device__ __forceinline__ explicit pk2(double c)
            : v(make_float2((float)c, (float)c))
        {
        }
    };
    __device__ __forceinline__ pk2 operator+(const pk2 a, const pk2 b)
    {
        return pk2(__fadd2_rn(a.v, b.v));
    }
    __device__ __forceinline__ pk2 operator-(const pk2 a, const pk2 b)
    {
        return pk2(__ffma2_rn(b.v, make_float2(-1.0f, -1.0f), a.v));
    }
    __device__ __forceinline__ pk2 operator*(const pk2 a, const pk2 b)
    {
        return pk2(__fmul2_rn(a.v, b.v));
    }
    __device__ __forceinline__ pk2 operator-(const pk2 a)
    {
        return pk2(__fmul2_rn(a.v, make_float2(-1.0f, -1.0f)));
    }
    template <>
    __device__ __forceinline__ pk2 bfma<pk2>(const pk2 a, const pk2 b, const pk2 c)
    {
        return pk2(__ffma2_rn(a.v, b.v, c.v));
    }
    template <>
    __device__ __forceinline__ pk2 madd<pk2>(const pk2 a, const pk2 c, const pk2 b, const pk2 s)
    {
        return pk2(__ffma2_rn(a.v, c.v, __fmul2_rn(b.v, s.v)));
    }
    template <>
    __device__ __forceinline__ pk2 msub<pk2>(const pk2 a, const pk2 c, const pk2 b, const pk2 s)
    {
        return pk2(__ffma2_rn(a.v, c.v, __fmul2_rn(b.v, make_float2(-s.v.x, -s.v.y))));
    }
    __device__ __forceinline__ pk2& operator*=(pk2& a, const pk2 b)
    {
        a = a * b;
        return a;
    }
    // complex value whose parts are packed pairs: two complex numbers, structure-of-arrays
    struct pk2c
    {
        pk2 x, y;
    };
    template <>
    struct cx<pk2>
    {
        using type = pk2c;
    };
#endif

    // type of a twiddle-table entry for values of component type T: the tables hold ordinary
    // complex numbers also when the data are packed pairs
    template <typename T>
    struct twof
    {
        using type = typename cx<T>::type;
    };
    // value times table entry
    template <typename T2>
    B200FFT_DEVICE T2 tmul(const T2 a, const T2 w)
    {
        return cmul(a, w);
    }
#if defined(__CUDACC__)
    template <>
    struct twof<pk2>
    {
        using type = float2;
    };
    // both complex numbers of the pair times the same table entry
    __device__ __forceinline__ pk2c tmul(const pk2c a, const float2 w)
    {
        const float2 wx = make_float2(w.x, w.x), wy = make_float2(w.y, w.y), nwy = make_float2(-w.y, -w.y);
        pk2c         r;
        r.x = pk2(__ffma2_rn(a.x.v, wx, __fmul2_rn(a.y.v, nwy)));
        r.y = pk2(__ffma2_rn(a.x.v, wy, __fmul2_rn(a.y.v, wx)));
        return r;
    }
#endif

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
