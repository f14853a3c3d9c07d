// Column-tile Stockham kernel for single precision in which every thread
// transforms TWO adjacent columns at once.
//
// Role in the reference: CS_KERNEL_STOCKHAM_BLOCK_CC
// (library/src/device/generator/stockham_gen_cc.h) — FFTs along a strided
// dimension with a tile of adjacent columns per workgroup so that global access
// stays coalesced.
//
// Why pairs: two neighbouring single-precision complex values are 16 bytes, so
// with a pair per thread every global and shared access is a 128-bit
// instruction, and the twiddle factor of a butterfly leg — identical for all
// columns — is loaded and applied once for two transforms.  On B200 the plain
// column kernel issues about 74 thread-instructions per point, which caps it
// near 70 % of HBM bandwidth; halving the memory and address instructions is
// what lifts that cap.
//
// Requirements checked by the planner / launch layer: unit stride across the
// tile's columns on both sides, even row pitches and outer strides, an even
// number of columns, 16-byte aligned bases (otherwise the plain column kernel
// runs).  An inverse transform is computed as conj(FFT(conj(x))): one sign
// flip on load, folded into the scale multiply on store.
#pragma once
#include "stockham_engine.cuh"

namespace b200fft
{
    template <class C>
    struct ColPair
    {
        static_assert(sizeof(typename C::T) == 4, "single precision only");
        static constexpr int NPAIR   = C::TPB / 2;
        static constexpr int THREADS = C::TPT * NPAIR;
        // rows are padded by one row every 16 so that stride-16 row patterns
        // fall on different halves of a 128-byte bank line
        static constexpr int    NROWS      = C::N + (C::N >> 4) + 1;
        static constexpr size_t SMEM_BYTES = (size_t)NROWS * NPAIR * sizeof(float4);
        __device__ static __forceinline__ int prow(int e)
        {
            return e + (e >> 4);
        }
        // padded row of (e0 + j * STRIDE); a compile-time constant offset from prow(e0)
        // whenever the stride is a multiple of 16
        template <int STRIDE>
        __device__ static __forceinline__ int prow_at(int e0, int pe0, int j)
        {
            if constexpr(STRIDE % 16 == 0)
                return pe0 + j * (STRIDE + STRIDE / 16);
            else
                return prow(e0 + j * STRIDE);
        }
    };

    template <class C, int P>
    struct ColPairPass
    {
        static constexpr int  W    = C::FL::get(P);
        static constexpr int  CH   = C::FL::cum(P);
        static constexpr int  NB   = C::N / W;
        static constexpr int  BPT  = (NB + C::TPT - 1) / C::TPT;
        static constexpr bool FULL = (NB % C::TPT) == 0;
        static constexpr int  TWO  = C::FL::tw_offset(P);
    };

    // twiddle + butterfly on the two columns held in xa / xb
    template <class C, int P>
    __device__ __forceinline__ void colpair_compute(float2 (&xa)[ColPairPass<C, P>::W],
                                                    float2 (&xb)[ColPairPass<C, P>::W],
                                                    const float2* __restrict__ tw,
                                                    int k)
    {
        using PP = ColPairPass<C, P>;
        if constexpr(P > 0)
        {
#pragma unroll
            for(int j = 1; j < PP::W; ++j)
            {
                const float2 w = tw[PP::TWO + (j - 1) * PP::CH + k];
                xa[j]          = cmul(xa[j], w);
                xb[j]          = cmul(xb[j], w);
            }
        }
        Butterfly<PP::W, float2>::run(xa);
        Butterfly<PP::W, float2>::run(xb);
    }

    // middle passes P .. NPASS-2: shared -> shared
    template <class C, int P>
    __device__ __forceinline__ void colpair_middle(int t, int cp, float4* sm, const float2* __restrict__ tw)
    {
        using CPK = ColPair<C>;
        using PP  = ColPairPass<C, P>;
        if constexpr(P < C::NPASS - 1)
        {
            float2 xa[PP::BPT][PP::W], xb[PP::BPT][PP::W];
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b = t + i * C::TPT;
                if(PP::FULL || b < PP::NB)
                {
                    const int pb = CPK::prow(b);
#pragma unroll
                    for(int j = 0; j < PP::W; ++j)
                    {
                        const float4 v = sm[CPK::template prow_at<PP::NB>(b, pb, j) * CPK::NPAIR + cp];
                        xa[i][j]       = make_float2(v.x, v.y);
                        xb[i][j]       = make_float2(v.z, v.w);
                    }
                }
            }
            __syncthreads();
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b = t + i * C::TPT;
                if(PP::FULL || b < PP::NB)
                {
                    const int k = b % PP::CH;
                    colpair_compute<C, P>(xa[i], xb[i], tw, k);
                    const int e0  = (b / PP::CH) * (PP::W * PP::CH) + k;
                    const int pe0 = CPK::prow(e0);
#pragma unroll
                    for(int j = 0; j < PP::W; ++j)
                        sm[CPK::template prow_at<PP::CH>(e0, pe0, j) * CPK::NPAIR + cp]
                            = make_float4(xa[i][j].x, xa[i][j].y, xb[i][j].x, xb[i][j].y);
                }
            }
            __syncthreads();
            colpair_middle<C, P + 1>(t, cp, sm, tw);
        }
    }

    // BLK: output with the two-level stride of b200fft_ioview::blk
    template <class C, bool BLK>
    __global__ void __launch_bounds__(ColPair<C>::THREADS, C::MINB)
        stockham_colpair_kernel(const __grid_constant__ b200fft_kargs a)
    {
        using CPK = ColPair<C>;
        static_assert(C::NPASS >= 2, "needs at least two passes");
        extern __shared__ __align__(16) unsigned char smem_raw[];
        float4* sm = reinterpret_cast<float4*>(smem_raw);

        const int     tid = threadIdx.x;
        const int     cp  = tid % CPK::NPAIR;
        const int     t   = tid / CPK::NPAIR;
        const TilePos tp  = decode_tile(a, blockIdx.x, C::TPB);
        const unsigned nvalid = min((unsigned)C::TPB, a.on[0] - tp.i0_first);
        const bool     valid  = (unsigned)(2 * cp) < nvalid;
        const float2* __restrict__ tw = reinterpret_cast<const float2*>(a.twiddles);

        const float sgn = a.inverse ? -1.0f : 1.0f; // conj on load
        const float sx  = a.use_scale ? (float)a.scale : 1.0f;
        const float sy  = sx * sgn; // conj + scale on store

        // ---- pass 0: global -> registers -> shared ----
        {
            using PP = ColPairPass<C, 0>;
            const long long ibase = view_base(a.in, tp.i0_first + 2 * cp, tp.i1, tp.i2);
            const float4*   gin   = reinterpret_cast<const float4*>(reinterpret_cast<const float2*>(a.in.p[0]) + ibase);
            const long long es4   = a.in.es >> 1; // row pitch in float4 units
            float2          xa[PP::BPT][PP::W], xb[PP::BPT][PP::W];
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b = t + i * C::TPT;
                if(PP::FULL || b < PP::NB)
                {
                    const float4* p  = gin + (long long)b * es4;
                    const int     st = (int)(PP::NB * es4); // the planner keeps N * pitch below 2^31
#pragma unroll
                    for(int j = 0; j < PP::W; ++j)
                    {
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if(valid)
                            v = p[j * st];
                        xa[i][j] = make_float2(v.x, v.y * sgn);
                        xb[i][j] = make_float2(v.z, v.w * sgn);
                    }
                }
            }
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b = t + i * C::TPT;
                if(PP::FULL || b < PP::NB)
                {
                    colpair_compute<C, 0>(xa[i], xb[i], tw, 0);
                    const int e0  = b * PP::W;
                    const int pe0 = CPK::prow(e0);
#pragma unroll
                    for(int j = 0; j < PP::W; ++j)
                        sm[CPK::template prow_at<1>(e0, pe0, j) * CPK::NPAIR + cp]
                            = make_float4(xa[i][j].x, xa[i][j].y, xb[i][j].x, xb[i][j].y);
                }
            }
            __syncthreads();
        }

        colpair_middle<C, 1>(t, cp, sm, tw);

        // ---- last pass: shared -> registers -> global ----
        {
            constexpr int P = C::NPASS - 1;
            using PP        = ColPairPass<C, P>;
            const long long obase = view_base(a.out, tp.i0_first + 2 * cp, tp.i1, tp.i2);
            float2*         gout  = reinterpret_cast<float2*>(a.out.p[0]) + obase;
            float2          xa[PP::BPT][PP::W], xb[PP::BPT][PP::W];
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b = t + i * C::TPT;
                if(PP::FULL || b < PP::NB)
                {
                    const int pb = CPK::prow(b);
#pragma unroll
                    for(int j = 0; j < PP::W; ++j)
                    {
                        const float4 v = sm[CPK::template prow_at<PP::NB>(b, pb, j) * CPK::NPAIR + cp];
                        xa[i][j]       = make_float2(v.x, v.y);
                        xb[i][j]       = make_float2(v.z, v.w);
                    }
                }
            }
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b = t + i * C::TPT;
                if(PP::FULL || b < PP::NB)
                {
                    const int k = b % PP::CH;
                    colpair_compute<C, P>(xa[i], xb[i], tw, k);
                    const int e0 = (b / PP::CH) * (PP::W * PP::CH) + k;
                    if(valid)
                    {
                        float2*   q   = gout + (long long)e0 * a.out.es;
                        const int ost = (int)(PP::CH * a.out.es);
#pragma unroll
                        for(int j = 0; j < PP::W; ++j)
                        {
                            float2* dst = BLK ? blk_address<float2>(a.out, obase, e0 + j * PP::CH) : q + j * ost;
                            *reinterpret_cast<float4*>(dst)
                                = make_float4(xa[i][j].x * sx, xa[i][j].y * sy, xb[i][j].x * sx, xb[i][j].y * sy);
                        }
                    }
                }
            }
        }
    }

    template <class C, bool BLK>
    cudaError_t launch_colpair_kernel(const b200fft_kargs& a, unsigned long long ntiles, cudaStream_t stream)
    {
        using CPK                 = ColPair<C>;
        static std::atomic<bool> attr_done[64]; // zero-initialised; host threads may launch the same kernel concurrently
        int         dev           = 0;
        cudaGetDevice(&dev);
        auto kern = stockham_colpair_kernel<C, BLK>;
        if(CPK::SMEM_BYTES > 48 * 1024 && dev < 64 && !attr_done[dev])
        {
            cudaError_t e
                = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CPK::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            attr_done[dev] = true;
        }
        if(ntiles == 0)
            return cudaSuccess;
        if(ntiles > 0x7fffffffull)
            return cudaErrorInvalidConfiguration;
        kern<<<(unsigned)ntiles, CPK::THREADS, CPK::SMEM_BYTES, stream>>>(a);
        return cudaGetLastError();
    }
} // namespace b200fft
