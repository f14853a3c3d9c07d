// Column-tile Stockham kernel in which a thread-block CLUSTER of two CTAs shares
// one 128-byte-wide tile through distributed shared memory.
//
// Role in the reference: CS_KERNEL_STOCKHAM_BLOCK_CC
// (library/src/device/generator/stockham_gen_cc.h): FFTs along a strided
// dimension, a tile of adjacent columns per workgroup.
//
// Why a cluster.  On B200 a strided tile only moves at full HBM rate when its row
// segments are whole 128-byte lines (measured: 64-byte segments reach 58 % of the
// copy rate, 128-byte segments 90 %).  A 128-byte-wide tile of a 1024-point column
// FFT is 128 KB, so a single CTA holding it leaves no room for a second resident
// CTA and nothing overlaps its load / compute / store phases.  Here the tile is
// split by ROWS between the two CTAs of a cluster: CTA r keeps rows
// [r*N/2, (r+1)*N/2) in its own shared memory (64 KB + padding) and runs half of
// the butterflies of every pass.  With the autosort Stockham indexing, butterfly
// b of pass p writes rows (b div CH)*W*CH + (b mod CH) + j*CH: giving CTA r the
// butterflies [r*NB/2, (r+1)*NB/2) makes all of its writes local, and its reads
// b + j*NB come from CTA 0 for j < W/2 and from CTA 1 for j >= W/2 — a compile-time
// choice per leg — through ld.shared::cluster.  Two to three such CTAs (from
// different clusters, in different phases) fit an SM, global loads and stores are
// full lines, and passes are separated by cluster barriers.
//
// Requirements (planner / launch layer): power-of-two length, unit stride across
// columns on both sides, column count a multiple of the tile width (16 single /
// 8 double complex), strides multiples of 16 bytes, 16-byte aligned bases.
// Inverse transforms are conj(FFT(conj x)).
#pragma once
#include "stockham_colcommon.cuh"

namespace b200fft
{
    namespace ptx
    {
        __device__ __forceinline__ unsigned cluster_ctarank()
        {
            unsigned r;
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
            return r;
        }
        __device__ __forceinline__ void cluster_sync()
        {
            asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        }
        __device__ __forceinline__ unsigned mapa(unsigned smem_addr, unsigned rank)
        {
            unsigned r;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
            return r;
        }
        __device__ __forceinline__ float4 ld_cluster(unsigned addr, float4*)
        {
            float4 v;
            asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                         : "r"(addr)
                         : "memory");
            return v;
        }
        __device__ __forceinline__ double2 ld_cluster(unsigned addr, double2*)
        {
            double2 v;
            asm volatile("ld.shared::cluster.v2.f64 {%0, %1}, [%2];" : "=d"(v.x), "=d"(v.y) : "r"(addr) : "memory");
            return v;
        }
    }

    template <class C, int CL = 2>
    struct ColCluster
    {
        using T                      = typename C::T;
        using U                      = typename Unit16<T>::type;
        static constexpr int VEC     = Unit16<T>::VEC;
        static constexpr int UNITS   = 8;
        static constexpr int COLS    = UNITS * VEC;
        static constexpr int HT      = C::TPT / CL; // butterfly lanes per CTA
        static constexpr int THREADS = HT * UNITS;
        static constexpr int HN      = C::N / CL; // rows held by one CTA
        static constexpr int HROWS   = HN + (HN >> 4) + 1;
        static constexpr int EPT     = C::N / C::TPT;
        static constexpr size_t SMEM_BYTES = (size_t)HROWS * UNITS * 16;
        static_assert(C::TPT % CL == 0, "butterfly lanes must split evenly over the cluster");
        __device__ static __forceinline__ int prow(int e)
        {
            return e + (e >> 4);
        }
    };

    template <class C, int CL, int P>
    __device__ __forceinline__ void colcluster_compute(typename C::T2 (&r)[ColCluster<C, CL>::VEC][ColCluster<C, CL>::EPT],
                                                       const typename C::T2* __restrict__ tw,
                                                       const int b0)
    {
        using CC = ColCluster<C, CL>;
        using PP = ColWidePass<C, P>;
        using T2 = typename C::T2;
        static_assert(PP::FULL && PP::BPT * PP::W == CC::EPT, "every radix must divide the points per thread");
#pragma unroll
        for(int i = 0; i < PP::BPT; ++i)
        {
            const int k = (b0 + i * CC::HT) % PP::CH;
            if constexpr(P > 0)
            {
#pragma unroll
                for(int j = 1; j < PP::W; ++j)
                {
                    const T2 w = tw[PP::TWO + (j - 1) * PP::CH + k];
#pragma unroll
                    for(int v = 0; v < CC::VEC; ++v)
                        r[v][i * PP::W + j] = cmul(r[v][i * PP::W + j], w);
                }
            }
#pragma unroll
            for(int v = 0; v < CC::VEC; ++v)
                Butterfly<PP::W, T2>::run(*reinterpret_cast<T2(*)[PP::W]>(&r[v][i * PP::W]));
        }
    }

    // passes P .. NPASS-1; r holds the inputs of pass P
    template <class C, int CL, int P, bool BLK>
    __device__ __forceinline__ void colcluster_from(const int                  rank,
                                                    const int                  tl, // butterfly lane in this CTA
                                                    const int                  u,
                                                    typename ColCluster<C, CL>::U* sm,
                                                    const unsigned (&win)[CL], // cluster-window addresses of every part
                                                    const typename C::T2* __restrict__ tw,
                                                    typename C::T2 (&r)[ColCluster<C, CL>::VEC][ColCluster<C, CL>::EPT],
                                                    const b200fft_ioview&      out,
                                                    typename C::T2*            gout,
                                                    const long long            obase,
                                                    typename C::T              sx,
                                                    typename C::T              sy)
    {
        using CC = ColCluster<C, CL>;
        using PP = ColWidePass<C, P>;
        using T  = typename C::T;
        using T2 = typename C::T2;
        using U  = typename CC::U;
        // this CTA's butterflies of pass P: b = rank*NB/CL + tl + i*HT
        const int b0 = rank * (PP::NB / CL) + tl;
        colcluster_compute<C, CL, P>(r, tw, b0);
        if constexpr(P == C::NPASS - 1)
        {
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b   = b0 + i * CC::HT;
                const int k   = b % PP::CH;
                const int e0  = (b / PP::CH) * (PP::W * PP::CH) + k;
                T2*       q   = gout + (long long)e0 * out.es;
                const int ost = (int)(PP::CH * out.es);
#pragma unroll
                for(int j = 0; j < PP::W; ++j)
                {
                    T2 tmp[CC::VEC];
#pragma unroll
                    for(int v = 0; v < CC::VEC; ++v)
                        tmp[v] = r[v][i * PP::W + j];
                    T2* dst = BLK ? blk_address<T2>(out, obase, e0 + j * PP::CH) : q + j * ost;
                    *reinterpret_cast<U*>(dst) = Unit16<T>::pack(tmp, sx, sy);
                }
            }
        }
        else
        {
            using PN = ColWidePass<C, P + 1>;
            static_assert(PN::W % CL == 0, "radices after the first must be multiples of the cluster size");
            static_assert((C::N / (PP::W * PP::CH)) % CL == 0, "output blocks must split evenly over the cluster");
            // results of pass P -> this CTA's rows (all local)
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b  = b0 + i * CC::HT;
                const int k  = b % PP::CH;
                const int e0 = (b / PP::CH) * (PP::W * PP::CH) + k - rank * CC::HN;
#pragma unroll
                for(int j = 0; j < PP::W; ++j)
                {
                    T2 tmp[CC::VEC];
#pragma unroll
                    for(int v = 0; v < CC::VEC; ++v)
                        tmp[v] = r[v][i * PP::W + j];
                    sm[CC::prow(e0 + j * PP::CH) * CC::UNITS + u] = Unit16<T>::pack(tmp);
                }
            }
            ptx::cluster_sync();
            // inputs of pass P+1: rows b + j*NB; legs j < W/2 live in CTA 0, the others in CTA 1
            const int bn0 = rank * (PN::NB / CL) + tl;
#pragma unroll
            for(int i = 0; i < PN::BPT; ++i)
            {
                const int b = bn0 + i * CC::HT;
#pragma unroll
                for(int j = 0; j < PN::W; ++j)
                {
                    const int     owner = (CL * j) / PN::W; // compile-time after unrolling
                    const int     row   = b + j * PN::NB - owner * CC::HN;
                    const U       v16   = ptx::ld_cluster(
                        win[owner] + (unsigned)((CC::prow(row) * CC::UNITS + u) * 16), static_cast<U*>(nullptr));
                    T2 tmp[CC::VEC];
                    Unit16<T>::unpack(v16, tmp, (T)1);
#pragma unroll
                    for(int v = 0; v < CC::VEC; ++v)
                        r[v][i * PN::W + j] = tmp[v];
                }
            }
            // nobody may overwrite (or leave) before both CTAs have finished reading
            ptx::cluster_sync();
            colcluster_from<C, CL, P + 1, BLK>(rank, tl, u, sm, win, tw, r, out, gout, obase, sx, sy);
        }
    }

    template <class C, int CL, bool BLK>
    __global__ void __cluster_dims__(CL, 1, 1) __launch_bounds__(ColCluster<C, CL>::THREADS, C::MINB)
        stockham_colcluster_kernel(const __grid_constant__ b200fft_kargs a)
    {
        using CC = ColCluster<C, CL>;
        using T  = typename C::T;
        using T2 = typename C::T2;
        using U  = typename CC::U;
        using P0 = ColWidePass<C, 0>;
        static_assert(C::NPASS >= 2, "needs at least two passes");
        static_assert(P0::BPT == 1 && P0::FULL, "pass 0 must be one butterfly per thread");
        extern __shared__ __align__(128) unsigned char smem_raw[];
        U* sm = reinterpret_cast<U*>(smem_raw);

        const int tid  = threadIdx.x;
        const int u    = tid % CC::UNITS;
        const int tl   = tid / CC::UNITS;
        const int rank = (int)ptx::cluster_ctarank();
        const T2* __restrict__ tw = reinterpret_cast<const T2*>(a.twiddles);
        const T sgn = a.inverse ? (T)-1 : (T)1;
        const T sx  = a.use_scale ? (T)a.scale : (T)1;
        const T sy  = sx * sgn;

        unsigned win[CL];
        {
            const unsigned local = (unsigned)__cvta_generic_to_shared(sm);
#pragma unroll
            for(int q = 0; q < CL; ++q)
                win[q] = ptx::mapa(local, q);
        }

        const unsigned  tile  = blockIdx.x / CL;
        const TilePos   tp    = decode_tile(a, tile, CC::COLS);
        const long long es_u  = (a.in.es * (long long)sizeof(T2)) / 16;
        const long long ibase = view_base(a.in, tp.i0_first, tp.i1, tp.i2);
        const U*        gin   = reinterpret_cast<const U*>(reinterpret_cast<const T2*>(a.in.p[0]) + ibase) + u;
        const long long obase = view_base(a.out, tp.i0_first + u * CC::VEC, tp.i1, tp.i2);
        T2*             gout  = reinterpret_cast<T2*>(a.out.p[0]) + obase;

        // pass-0 inputs straight from global memory: butterfly b = rank*NB0/2 + tl, rows b + j*NB0
        T2 r[CC::VEC][CC::EPT];
        {
            const int b    = rank * (P0::NB / CL) + tl;
            const U*  src  = gin + (long long)b * es_u;
            const int step = (int)(P0::NB * es_u);
#pragma unroll
            for(int j = 0; j < P0::W; ++j)
            {
                T2 tmp[CC::VEC];
                Unit16<T>::unpack(src[(long long)j * step], tmp, sgn);
#pragma unroll
                for(int v = 0; v < CC::VEC; ++v)
                    r[v][j] = tmp[v];
            }
        }
        colcluster_from<C, CL, 0, BLK>(rank, tl, u, sm, win, tw, r, a.out, gout, obase, sx, sy);
    }

    template <class C, int CL, bool BLK>
    cudaError_t launch_colcluster_kernel(const b200fft_kargs& a, unsigned long long ntiles, cudaStream_t stream)
    {
        using CC                  = ColCluster<C, CL>;
        static std::atomic<bool> attr_done[64]; // zero-initialised; host threads may launch the same kernel concurrently
        int         dev           = 0;
        cudaGetDevice(&dev);
        auto kern = stockham_colcluster_kernel<C, CL, BLK>;
        if(CC::SMEM_BYTES > 48 * 1024 && dev < 64 && !attr_done[dev])
        {
            cudaError_t e
                = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CC::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            attr_done[dev] = true;
        }
        if(ntiles == 0)
            return cudaSuccess;
        if(CL * ntiles > 0x7fffffffull)
            return cudaErrorInvalidConfiguration;
        kern<<<(unsigned)(CL * ntiles), CC::THREADS, CC::SMEM_BYTES, stream>>>(a);
        return cudaGetLastError();
    }
} // namespace b200fft
