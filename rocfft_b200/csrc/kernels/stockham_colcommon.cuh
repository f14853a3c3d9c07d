// Pieces shared by the column kernels whose tiles are 128 bytes wide (stockham_colcluster.cuh,
// stockham_colpush.cuh, stockham_colstream.cuh): the 16-byte unit a thread moves per row — two
// single or one double complex column — and the compile-time constants of one radix pass.
//
// Role in the reference: the per-pass constants correspond to the width / cumulative-height /
// butterfly-count bookkeeping of library/src/device/generator/stockham_gen_base.h:642-764.
#pragma once
#include "stockham_engine.cuh"

namespace b200fft
{
    template <typename T>
    struct Unit16;
    template <>
    struct Unit16<float>
    {
        using type               = float4;
        static constexpr int VEC = 2;
        __device__ static __forceinline__ void unpack(const float4 v, float2 (&x)[2], float sgn)
        {
            x[0] = make_float2(v.x, v.y * sgn);
            x[1] = make_float2(v.z, v.w * sgn);
        }
        __device__ static __forceinline__ float4 pack(const float2 (&x)[2], float sx, float sy)
        {
            return make_float4(x[0].x * sx, x[0].y * sy, x[1].x * sx, x[1].y * sy);
        }
        __device__ static __forceinline__ float4 pack(const float2 (&x)[2])
        {
            return make_float4(x[0].x, x[0].y, x[1].x, x[1].y);
        }
    };
    template <>
    struct Unit16<double>
    {
        using type               = double2;
        static constexpr int VEC = 1;
        __device__ static __forceinline__ void unpack(const double2 v, double2 (&x)[1], double sgn)
        {
            x[0] = make_double2(v.x, v.y * sgn);
        }
        __device__ static __forceinline__ double2 pack(const double2 (&x)[1], double sx, double sy)
        {
            return make_double2(x[0].x * sx, x[0].y * sy);
        }
        __device__ static __forceinline__ double2 pack(const double2 (&x)[1])
        {
            return x[0];
        }
    };

    template <class C, int P>
    struct ColWidePass
    {
        static constexpr int  W    = C::FL::get(P);
        static constexpr int  CH   = C::FL::cum(P);
        static constexpr int  NB   = C::N / W;
        static constexpr int  BPT  = (NB + C::TPT - 1) / C::TPT;
        static constexpr bool FULL = (NB % C::TPT) == 0;
        static constexpr int  TWO  = C::FL::tw_offset(P);
    };
} // namespace b200fft
