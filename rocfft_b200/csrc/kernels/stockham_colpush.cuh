// Column-tile Stockham kernel in which a thread-block CLUSTER shares one
// 128-byte-wide tile and exchanges it between passes with asynchronous
// remote stores (st.async + mbarrier transaction counts).
//
// Role in the reference: CS_KERNEL_STOCKHAM_BLOCK_CC
// (library/src/device/generator/stockham_gen_cc.h): FFTs along a strided
// dimension, a tile of adjacent columns per workgroup.
//
// Why a cluster.  A strided tile only moves at full HBM rate when its row
// segments are whole 128-byte lines, and a 128-byte-wide tile of a 1024-point
// column FFT is 128 KB: one CTA holding it leaves no room for a second resident
// CTA.  Here the tile is split between the CL CTAs of a cluster (64 KB each for
// CL = 2), so two CTAs of different clusters fit an SM.
//
// Why pushes.  Between two passes every point changes owner.  Reading the peer's
// shared memory (ld.shared::cluster) needs a release/acquire cluster barrier after
// the writes AND a full barrier after the reads, and the release showed up as the
// largest stall of that design (membar, 3.8 warp-cycles per issue).  Here the
// producer pushes instead: after pass P every thread sends its results with
// st.async straight into the shared memory of the CTA that will consume them in
// pass P+1; each store credits its bytes to the consumer's mbarrier, the consumer
// waits for the byte count of its part of the tile and then reads LOCAL shared
// memory.  No fence is needed for the data.  Before the next exchange the buffers
// must be free again: every CTA arrives (relaxed) on the hardware cluster barrier
// once its local reads are issued and waits on it just before it pushes again, so
// the barrier latency hides behind the butterflies of pass P+1.
//
// Ownership.  Pass Q reads rows b + j*NB_Q (NB_Q = N / W_Q).  CTA r runs the
// butterflies b in [r*NB_Q/CL, (r+1)*NB_Q/CL) and therefore owns the rows e with
// (e mod NB_Q) in that range; they are stored densely at local row
// (e div NB_Q)*(NB_Q/CL) + (e mod NB_Q) - r*NB_Q/CL.
//
// Requirements (planner / launch layer): power-of-two length, unit stride across
// columns on both sides, column count a multiple of the tile width (16 single /
// 8 double complex), strides multiples of 16 bytes, 16-byte aligned bases.
// Inverse transforms are conj(FFT(conj x)).  Every mbarrier wait is bounded; on
// expiry the kernel raises the plan's device error flag (aux[3]) and carries on,
// so that the cluster still leaves in step.  No multicast and no TMA: the kernel
// is legal in multi-GPU runs.
#pragma once
#include "stockham_colcluster.cuh"
#include "stockham_rows_tma.cuh"

namespace b200fft
{
    namespace ptx
    {
        __device__ __forceinline__ void cluster_arrive_relaxed()
        {
            asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
        }
        __device__ __forceinline__ void cluster_arrive_release()
        {
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        }
        __device__ __forceinline__ void cluster_wait()
        {
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        }
        // 16-byte asynchronous store into a (possibly remote) CTA's shared memory; the bytes
        // are credited to the mbarrier at `bar` (an address in the same CTA's window)
        __device__ __forceinline__ void st_async16(unsigned addr, const float4 v, unsigned bar)
        {
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(
                             addr),
                         "f"(v.x),
                         "f"(v.y),
                         "f"(v.z),
                         "f"(v.w),
                         "r"(bar)
                         : "memory");
        }
        __device__ __forceinline__ void st_async16(unsigned addr, const double2 v, unsigned bar)
        {
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f64 [%0], {%1, %2}, [%3];" ::"r"(addr),
                         "d"(v.x),
                         "d"(v.y),
                         "r"(bar)
                         : "memory");
        }
    }

    template <class C, int CL = 2>
    struct ColPush
    {
        using T                      = typename C::T;
        using U                      = typename Unit16<T>::type;
        static constexpr int VEC     = Unit16<T>::VEC;
        static constexpr int UNITS   = 8; // 16-byte units per 128-byte row segment
        static constexpr int COLS    = UNITS * VEC;
        static constexpr int HT      = C::TPT / CL; // butterfly lanes per CTA
        static constexpr int THREADS = HT * UNITS;
        static constexpr int HN      = C::N / CL; // rows held by one CTA
        static constexpr int EPT     = C::N / C::TPT;
        static constexpr unsigned PART_BYTES = (unsigned)HN * UNITS * 16;
        static constexpr size_t   SMEM_BYTES = (size_t)PART_BYTES + 16; // + the mbarrier
        static_assert(C::TPT % CL == 0, "butterfly lanes must split evenly over the cluster");
        static_assert((C::N & (C::N - 1)) == 0, "power-of-two lengths only");
    };

    template <class C, int CL, int P>
    __device__ __forceinline__ void colpush_compute(typename C::T2 (&r)[ColPush<C, CL>::VEC][ColPush<C, CL>::EPT],
                                                    const typename C::T2* __restrict__ tw,
                                                    const int b0)
    {
        using CC = ColPush<C, CL>;
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
    __device__ __forceinline__ void colpush_from(const int               rank,
                                                 const int               tl, // butterfly lane in this CTA
                                                 const int               u,
                                                 const typename ColPush<C, CL>::U* sm,
                                                 uint64_t*               bar,
                                                 const unsigned (&win)[CL], // cluster-window addresses of every part
                                                 const unsigned (&wbar)[CL], // ... and of every part's mbarrier
                                                 const typename C::T2* __restrict__ tw,
                                                 typename C::T2 (&r)[ColPush<C, CL>::VEC][ColPush<C, CL>::EPT],
                                                 const b200fft_kargs&    a,
                                                 typename C::T2*         gout,
                                                 const long long         obase,
                                                 typename C::T           sx,
                                                 typename C::T           sy)
    {
        using CC = ColPush<C, CL>;
        using PP = ColWidePass<C, P>;
        using T  = typename C::T;
        using T2 = typename C::T2;
        using U  = typename CC::U;
        // this CTA's butterflies of pass P: b = rank*NB/CL + tl + i*HT
        const int b0 = rank * (PP::NB / CL) + tl;
        colpush_compute<C, CL, P>(r, tw, b0);
        if constexpr(P == C::NPASS - 1)
        {
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b   = b0 + i * CC::HT;
                const int k   = b % PP::CH;
                const int e0  = (b / PP::CH) * (PP::W * PP::CH) + k;
                T2*       q   = gout + (long long)e0 * a.out.es;
                const int ost = (int)(PP::CH * a.out.es);
#pragma unroll
                for(int j = 0; j < PP::W; ++j)
                {
                    T2 tmp[CC::VEC];
#pragma unroll
                    for(int v = 0; v < CC::VEC; ++v)
                        tmp[v] = r[v][i * PP::W + j];
                    T2* dst = BLK ? blk_address<T2>(a.out, obase, e0 + j * PP::CH) : q + j * ost;
                    *reinterpret_cast<U*>(dst) = Unit16<T>::pack(tmp, sx, sy);
                }
            }
        }
        else
        {
            using PN          = ColWidePass<C, P + 1>;
            constexpr int NBQ = PN::NB; // row e is consumed by butterfly (e mod NBQ) of pass P+1
            constexpr int PER = NBQ / CL; // butterflies of pass P+1 per CTA
            static_assert(NBQ % CL == 0 && PER % CC::HT == 0, "next pass must split evenly over the cluster");
            // P > 0: every CTA of the cluster has taken its inputs of pass P out of its buffer;
            // P = 0: every CTA has initialised its mbarrier (arrival at the top of the kernel)
            ptx::cluster_wait();
            if(threadIdx.x == 0)
                ptx::mbar_expect_tx(bar, CC::PART_BYTES);
            // results of pass P -> the buffers of the CTAs that consume them
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b  = b0 + i * CC::HT;
                const int k  = b % PP::CH;
                const int e0 = (b / PP::CH) * (PP::W * PP::CH) + k;
#pragma unroll
                for(int j = 0; j < PP::W; ++j)
                {
                    T2 tmp[CC::VEC];
#pragma unroll
                    for(int v = 0; v < CC::VEC; ++v)
                        tmp[v] = r[v][i * PP::W + j];
                    const int      e     = e0 + j * PP::CH;
                    const int      rem   = e % NBQ;
                    const int      owner = rem / PER;
                    const int      lrow  = (e / NBQ) * PER + (rem - owner * PER);
                    const unsigned off   = (unsigned)((lrow * CC::UNITS + u) * 16);
                    unsigned       dst = win[0], dbar = wbar[0];
#pragma unroll
                    for(int q = 1; q < CL; ++q)
                    {
                        dst  = owner == q ? win[q] : dst;
                        dbar = owner == q ? wbar[q] : dbar;
                    }
                    ptx::st_async16(dst + off, Unit16<T>::pack(tmp), dbar);
                }
            }
            // all PART_BYTES of this CTA's part have landed
            if(!ptx::mbar_wait(bar, (unsigned)(P & 1)))
            {
                if(a.aux[3])
                    atomicExch(reinterpret_cast<int*>(const_cast<void*>(a.aux[3])), 1);
            }
            // inputs of pass P+1: butterfly b = rank*PER + tl + i*HT reads rows b + j*NBQ,
            // stored at local rows j*PER + tl + i*HT
#pragma unroll
            for(int i = 0; i < PN::BPT; ++i)
            {
#pragma unroll
                for(int j = 0; j < PN::W; ++j)
                {
                    const U v16 = sm[(j * PER + tl + i * CC::HT) * CC::UNITS + u];
                    T2      tmp[CC::VEC];
                    Unit16<T>::unpack(v16, tmp, (T)1);
#pragma unroll
                    for(int v = 0; v < CC::VEC; ++v)
                        r[v][i * PN::W + j] = tmp[v];
                }
            }
            // the buffer may be refilled once every CTA has got here; waited for before the next push.
            // Release semantics order the shared-memory reads above before the peers' next pushes
            // into the same slots (only kernels of three or more passes get here).
            if constexpr(P + 1 < C::NPASS - 1)
                ptx::cluster_arrive_release();
            colpush_from<C, CL, P + 1, BLK>(rank, tl, u, sm, bar, win, wbar, tw, r, a, gout, obase, sx, sy);
        }
    }

    template <class C, int CL, bool BLK>
    __global__ void __cluster_dims__(CL, 1, 1) __launch_bounds__(ColPush<C, CL>::THREADS, C::MINB)
        stockham_colpush_kernel(const __grid_constant__ b200fft_kargs a)
    {
        using CC = ColPush<C, CL>;
        using T  = typename C::T;
        using T2 = typename C::T2;
        using U  = typename CC::U;
        using P0 = ColWidePass<C, 0>;
        static_assert(C::NPASS >= 2, "needs at least two passes");
        static_assert(P0::BPT == 1 && P0::FULL, "pass 0 must be one butterfly per thread");
        extern __shared__ __align__(128) unsigned char smem_raw[];
        U*        sm  = reinterpret_cast<U*>(smem_raw);
        uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw + CC::PART_BYTES);

        const int tid  = threadIdx.x;
        const int u    = tid % CC::UNITS;
        const int tl   = tid / CC::UNITS;
        const int rank = (int)ptx::cluster_ctarank();
        const T2* __restrict__ tw = reinterpret_cast<const T2*>(a.twiddles);
        const T sgn = a.inverse ? (T)-1 : (T)1;
        const T sx  = a.use_scale ? (T)a.scale : (T)1;
        const T sy  = sx * sgn;

        unsigned win[CL], wbar[CL];
        {
            const unsigned local = ptx::smem_u32(sm);
            const unsigned lbar  = ptx::smem_u32(bar);
#pragma unroll
            for(int q = 0; q < CL; ++q)
            {
                win[q]  = ptx::mapa(local, q);
                wbar[q] = ptx::mapa(lbar, q);
            }
        }
        if(tid == 0)
        {
            ptx::mbar_init(bar, 1);
            ptx::fence_mbar_init();
        }
        // every mbarrier of the cluster must be initialised before anybody pushes: the init is
        // published by fence.mbarrier_init, so a relaxed arrival suffices; the matching wait
        // stands before the first push, behind the global loads and the butterflies of pass 0
        ptx::cluster_arrive_relaxed();

        const unsigned  tile  = blockIdx.x / CL;
        const TilePos   tp    = decode_tile(a, tile, CC::COLS);
        const long long es_u  = (a.in.es * (long long)sizeof(T2)) / 16;
        const long long ibase = view_base(a.in, tp.i0_first, tp.i1, tp.i2);
        const U*        gin   = reinterpret_cast<const U*>(reinterpret_cast<const T2*>(a.in.p[0]) + ibase) + u;
        const long long obase = view_base(a.out, tp.i0_first + u * CC::VEC, tp.i1, tp.i2);
        T2*             gout  = reinterpret_cast<T2*>(a.out.p[0]) + obase;

        // pass-0 inputs straight from global memory: butterfly b = rank*NB0/CL + tl, rows b + j*NB0
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
        colpush_from<C, CL, 0, BLK>(rank, tl, u, sm, bar, win, wbar, tw, r, a, gout, obase, sx, sy);
    }

    template <class C, int CL, bool BLK>
    cudaError_t launch_colpush_kernel(const b200fft_kargs& a, unsigned long long ntiles, cudaStream_t stream)
    {
        using CC                  = ColPush<C, CL>;
        static std::atomic<bool> attr_done[64]; // zero-initialised; host threads may launch the same kernel concurrently
        int         dev           = 0;
        cudaGetDevice(&dev);
        auto kern = stockham_colpush_kernel<C, CL, BLK>;
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
