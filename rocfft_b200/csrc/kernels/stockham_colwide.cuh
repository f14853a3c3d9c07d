// Column-tile Stockham kernel with full-cache-line tiles, a persistent CTA per SM
// and asynchronous prefetch of the next tile.
//
// Role in the reference: CS_KERNEL_STOCKHAM_BLOCK_CC
// (library/src/device/generator/stockham_gen_cc.h): FFTs along a strided
// dimension, a tile of adjacent columns per workgroup.
//
// Why this shape.  Measured on B200, a strided tile moves at a rate set by the
// width of its row segments: 32 B -> 28 %, 64 B -> 58 %, 128 B -> 90 % of the HBM
// copy rate.  A column tile must therefore be 128 bytes wide (16 single or 8
// double complex columns).  For N = 1024 that is a 128 KB tile: only one fits an
// SM, so overlap of loading, computing and storing cannot come from several
// resident CTAs.  Instead:
//   * the CTA is persistent and fetches tile i+1 with cp.async (16 bytes per
//     thread, eight threads per 128-byte line) into a raw staging buffer while it
//     transforms tile i;
//   * tile i lives in registers (every thread owns one 16-byte unit — two single
//     or one double complex column — of its butterflies) and passes exchange
//     data through a shared buffer that holds only HALF of the tile: the two
//     halves of each row (units 0-3, units 4-7) take turns, which is what makes
//     staging buffer + exchange buffer fit in 227 KB;
//   * results are stored from registers as full 128-byte lines.
// Inverse transforms are conj(FFT(conj x)): a sign flip on load, folded into
// the scale on store.
//
// Requirements (planner / launch layer): unit stride across columns on both
// sides, column count a multiple of the tile width, row pitches and outer
// strides multiples of 16 bytes, 16-byte aligned bases; otherwise the plain
// column kernel runs.
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

    template <class C>
    struct ColWide
    {
        using T                      = typename C::T;
        using U                      = typename Unit16<T>::type;
        static constexpr int VEC     = Unit16<T>::VEC;
        static constexpr int UNITS   = 8; // 16-byte units per 128-byte row segment
        static constexpr int HALF    = 4;
        static constexpr int COLS    = UNITS * VEC; // columns per tile
        static constexpr int THREADS = C::TPT * UNITS;
        static constexpr int XROWS   = C::N + (C::N >> 4) + 1; // exchange rows, padded
        static constexpr size_t STAGE_BYTES = (size_t)C::N * UNITS * 16;
        static constexpr size_t XCHG_BYTES  = (size_t)XROWS * HALF * 16;
        static constexpr size_t SMEM_BYTES  = STAGE_BYTES + XCHG_BYTES;
        __device__ static __forceinline__ int prow(int e)
        {
            return e + (e >> 4);
        }
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
    struct ColWidePass
    {
        static constexpr int  W    = C::FL::get(P);
        static constexpr int  CH   = C::FL::cum(P);
        static constexpr int  NB   = C::N / W;
        static constexpr int  BPT  = (NB + C::TPT - 1) / C::TPT;
        static constexpr bool FULL = (NB % C::TPT) == 0;
        static constexpr int  TWO  = C::FL::tw_offset(P);
    };

    // All passes work on one flat register array r[VEC][EPT] (EPT = N / TPT points per
    // thread and column); pass P views it as BPT butterflies of W points:
    // butterfly i, leg j  <->  r[v][i * W + j].  Every radix must divide EPT.
    template <class C, int P>
    __device__ __forceinline__ void colwide_compute(typename C::T2 (&r)[ColWide<C>::VEC][C::N / C::TPT],
                                                    const typename C::T2* __restrict__ tw,
                                                    const int t)
    {
        using PP = ColWidePass<C, P>;
        using T2 = typename C::T2;
        static_assert(PP::FULL && PP::BPT * PP::W == C::N / C::TPT, "every radix must divide the points per thread");
#pragma unroll
        for(int i = 0; i < PP::BPT; ++i)
        {
            const int k = (t + i * C::TPT) % PP::CH;
            if constexpr(P > 0)
            {
#pragma unroll
                for(int j = 1; j < PP::W; ++j)
                {
                    const T2 w = tw[PP::TWO + (j - 1) * PP::CH + k];
#pragma unroll
                    for(int v = 0; v < ColWide<C>::VEC; ++v)
                        r[v][i * PP::W + j] = cmul(r[v][i * PP::W + j], w);
                }
            }
#pragma unroll
            for(int v = 0; v < ColWide<C>::VEC; ++v)
                Butterfly<PP::W, T2>::run(*reinterpret_cast<T2(*)[PP::W]>(&r[v][i * PP::W]));
        }
    }

    // Exchange between pass P (results in r) and pass P+1 (inputs into r, in place) through
    // the half-tile buffer: units 0-3 first, then units 4-7.
    template <class C, int P>
    __device__ __forceinline__ void colwide_exchange(const int                t,
                                                     const int                u,
                                                     typename ColWide<C>::U*  xch,
                                                     typename C::T2 (&r)[ColWide<C>::VEC][C::N / C::TPT])
    {
        using CW = ColWide<C>;
        using PS = ColWidePass<C, P>;
        using PL = ColWidePass<C, P + 1>;
        using T  = typename C::T;
        const int uh = u & 3;
#pragma unroll
        for(int g = 0; g < 2; ++g)
        {
            if((u >> 2) == g)
            {
#pragma unroll
                for(int i = 0; i < PS::BPT; ++i)
                {
                    const int b   = t + i * C::TPT;
                    const int k   = b % PS::CH;
                    const int e0  = (b / PS::CH) * (PS::W * PS::CH) + k;
                    const int pe0 = CW::prow(e0);
#pragma unroll
                    for(int j = 0; j < PS::W; ++j)
                    {
                        typename C::T2 tmp[CW::VEC];
#pragma unroll
                        for(int v = 0; v < CW::VEC; ++v)
                            tmp[v] = r[v][i * PS::W + j];
                        xch[CW::template prow_at<PS::CH>(e0, pe0, j) * CW::HALF + uh] = Unit16<T>::pack(tmp);
                    }
                }
            }
            __syncthreads();
            if((u >> 2) == g)
            {
#pragma unroll
                for(int i = 0; i < PL::BPT; ++i)
                {
                    const int b  = t + i * C::TPT;
                    const int pb = CW::prow(b);
#pragma unroll
                    for(int j = 0; j < PL::W; ++j)
                    {
                        typename C::T2 tmp[CW::VEC];
                        Unit16<T>::unpack(xch[CW::template prow_at<PL::NB>(b, pb, j) * CW::HALF + uh], tmp, (T)1);
#pragma unroll
                        for(int v = 0; v < CW::VEC; ++v)
                            r[v][i * PL::W + j] = tmp[v];
                    }
                }
            }
            __syncthreads();
        }
    }

    // passes P .. NPASS-1 with the inputs of pass P already in r
    template <class C, int P, bool BLK>
    __device__ __forceinline__ void colwide_from(const int               t,
                                                 const int               u,
                                                 typename ColWide<C>::U* xch,
                                                 const typename C::T2* __restrict__ tw,
                                                 typename C::T2 (&r)[ColWide<C>::VEC][C::N / C::TPT],
                                                 const b200fft_ioview&   out,
                                                 typename C::T2*         gout,
                                                 const long long         obase,
                                                 typename C::T           sx,
                                                 typename C::T           sy)
    {
        using CW = ColWide<C>;
        using PP = ColWidePass<C, P>;
        using T  = typename C::T;
        using T2 = typename C::T2;
        colwide_compute<C, P>(r, tw, t);
        if constexpr(P == C::NPASS - 1)
        {
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b   = t + i * C::TPT;
                const int k   = b % PP::CH;
                const int e0  = (b / PP::CH) * (PP::W * PP::CH) + k;
                T2*       q   = gout + (long long)e0 * out.es;
                const int ost = (int)(PP::CH * out.es);
#pragma unroll
                for(int j = 0; j < PP::W; ++j)
                {
                    T2 tmp[CW::VEC];
#pragma unroll
                    for(int v = 0; v < CW::VEC; ++v)
                        tmp[v] = r[v][i * PP::W + j];
                    T2* dst = BLK ? blk_address<T2>(out, obase, e0 + j * PP::CH) : q + j * ost;
                    *reinterpret_cast<typename CW::U*>(dst) = Unit16<T>::pack(tmp, sx, sy);
                }
            }
        }
        else
        {
            colwide_exchange<C, P>(t, u, xch, r);
            colwide_from<C, P + 1, BLK>(t, u, xch, tw, r, out, gout, obase, sx, sy);
        }
    }

    template <class C, bool BLK>
    __global__ void __launch_bounds__(ColWide<C>::THREADS, 1)
        stockham_colwide_kernel(const __grid_constant__ b200fft_kargs a)
    {
        using CW = ColWide<C>;
        using T  = typename C::T;
        using T2 = typename C::T2;
        using U  = typename CW::U;
        using P0 = ColWidePass<C, 0>;
        static_assert(C::NPASS >= 2, "needs at least two passes");
        static_assert(P0::BPT == 1 && P0::FULL, "pass 0 must be one butterfly per thread");
        extern __shared__ __align__(128) unsigned char smem_raw[];
        U* stage = reinterpret_cast<U*>(smem_raw);
        U* xch   = reinterpret_cast<U*>(smem_raw + CW::STAGE_BYTES);

        const int tid = threadIdx.x;
        const int u   = tid % CW::UNITS;
        const int t   = tid / CW::UNITS;
        const T2* __restrict__ tw = reinterpret_cast<const T2*>(a.twiddles);
        const T sgn = a.inverse ? (T)-1 : (T)1;
        const T sx  = a.use_scale ? (T)a.scale : (T)1;
        const T sy  = sx * sgn;

        const unsigned long long ntiles = (unsigned long long)a.ntile0 * a.on[1] * a.on[2];
        const long long es_u = (a.in.es * (long long)sizeof(T2)) / 16; // row pitch in 16-byte units

        // cp.async of one tile: chunk q = tid + k*THREADS, row q / 8, unit q % 8
        auto prefetch = [&](unsigned long long tile) {
            const TilePos   tp   = decode_tile(a, (unsigned)tile, CW::COLS);
            const long long base = view_base(a.in, tp.i0_first, tp.i1, tp.i2);
            const U*        g    = reinterpret_cast<const U*>(reinterpret_cast<const T2*>(a.in.p[0]) + base) + u;
            constexpr int ROWS_PER_STEP = CW::THREADS / CW::UNITS;
            constexpr int STEPS         = C::N / ROWS_PER_STEP;
            const U*      src           = g + (long long)t * es_u;
            const int     step          = (int)(ROWS_PER_STEP * es_u);
            unsigned      dst = (unsigned)__cvta_generic_to_shared(stage + (size_t)t * CW::UNITS + u);
#pragma unroll
            for(int k = 0; k < STEPS; ++k)
            {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + k * ROWS_PER_STEP * CW::UNITS * 16),
                             "l"(src + (long long)k * step)
                             : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };

        unsigned long long tile = blockIdx.x;
        if(tile < ntiles)
            prefetch(tile);
        for(; tile < ntiles; tile += gridDim.x)
        {
            // every thread reads back exactly the chunks it copied itself (rows t + j*NB0 of
            // unit u), so waiting for its own copies is all the synchronisation the staging
            // buffer needs
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            T2 x[CW::VEC][C::N / C::TPT];
#pragma unroll
            for(int j = 0; j < P0::W; ++j)
            {
                T2 tmp[CW::VEC];
                Unit16<T>::unpack(stage[(size_t)(t + j * P0::NB) * CW::UNITS + u], tmp, sgn);
#pragma unroll
                for(int v = 0; v < CW::VEC; ++v)
                    x[v][j] = tmp[v];
            }
            const unsigned long long next = tile + gridDim.x;
            if(next < ntiles)
                prefetch(next);

            const TilePos   tp    = decode_tile(a, (unsigned)tile, CW::COLS);
            const long long obase = view_base(a.out, tp.i0_first + u * CW::VEC, tp.i1, tp.i2);
            T2*             gout  = reinterpret_cast<T2*>(a.out.p[0]) + obase;
            colwide_from<C, 0, BLK>(t, u, xch, tw, x, a.out, gout, obase, sx, sy);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }

    template <class C, bool BLK>
    cudaError_t launch_colwide_kernel(const b200fft_kargs& a, unsigned long long ntiles, cudaStream_t stream)
    {
        using CW                     = ColWide<C>;
        static int blocks_per_sm[64] = {};
        static int sm_count[64]      = {};
        int        dev               = 0;
        cudaGetDevice(&dev);
        if(dev >= 64)
            return cudaErrorInvalidDevice;
        auto kern = stockham_colwide_kernel<C, BLK>;
        if(!blocks_per_sm[dev])
        {
            cudaError_t e
                = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CW::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            int nb = 0;
            e      = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kern, CW::THREADS, CW::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
            blocks_per_sm[dev] = nb > 0 ? nb : 1;
        }
        if(ntiles == 0)
            return cudaSuccess;
        if(ntiles > 0x7fffffffull)
            return cudaErrorInvalidConfiguration;
        unsigned long long grid = (unsigned long long)blocks_per_sm[dev] * sm_count[dev];
        if(grid > ntiles)
            grid = ntiles;
        kern<<<(unsigned)grid, CW::THREADS, CW::SMEM_BYTES, stream>>>(a);
        return cudaGetLastError();
    }
} // namespace b200fft
