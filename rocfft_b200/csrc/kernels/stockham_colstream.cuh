// Persistent column-tile Stockham kernel fed by the tensor copy engine (TMA).
//
// Role in the reference: CS_KERNEL_STOCKHAM_BLOCK_CC
// (library/src/device/generator/stockham_gen_cc.h; chosen for the higher
// dimensions of 2D/3D transforms, library/src/tree_node_1D.cpp:1102-1112): FFTs
// along a strided dimension, a tile of adjacent columns per workgroup.
//
// Shape.  A tile is N rows x 128 bytes (16 single or 8 double complex columns):
// strided tiles only move at the full HBM rate when their row segments are whole
// 128-byte lines.  One persistent CTA per resident slot walks over the tiles:
//
//   load     one elected thread issues cp.async.bulk.tensor box loads (boxes of up to
//            256 rows x 128 bytes, described by a tensor map of the caller's array;
//            no multicast, no cluster) that land in a shared-memory stage and
//            complete on an mbarrier — no thread holds registers for data in flight;
//   pass 0   every thread moves its points from the stage into registers; after one
//            barrier the stage is free and the load of the CTA's NEXT tile is issued,
//            so it is in flight during everything that follows;
//   exchange between passes the tile changes owner through a shared buffer that holds
//            half of it: real parts first, imaginary parts second;
//   store    the last pass writes its results from registers straight to global
//            memory as 16-byte units (whole 128-byte lines per row).
//
// Single precision runs TWO adjacent columns per thread in packed form (pk2c: real
// parts of both columns in one aligned register pair, imaginary parts in another), so
// every butterfly instruction is a packed fp32 instruction serving two transforms; a
// 16-byte unit of a row is exactly one such pair of complex values.  Double precision
// runs one column per thread.  Either way a value's component is 8 bytes, which is
// what the exchange buffer is made of.
//
// Requirements (planner / launch layer): power-of-two length, unit stride across
// columns on both sides, column count a multiple of the tile width, input strides
// positive multiples of 16 bytes, 16-byte aligned bases.  Inverse transforms are
// conj(FFT(conj x)).  Every mbarrier wait is bounded; when one gives up, the whole CTA
// learns of it at the next barrier, raises the plan's device error flag (aux[3]), waits
// (bounded again) for the copy that is still in flight and leaves.
#pragma once
#include "stockham_colpush.cuh"
#include <cuda.h>
#include <cstdlib>
#include <mutex>
#include <utility>

namespace b200fft
{
    namespace ptx
    {
        // 4D tiled box load, global -> shared, completing on an mbarrier of this CTA (no multicast)
        __device__ __forceinline__ void
            tma_load_4d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar)
        {
            asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, "
                         "%4, %5}], [%6];" ::"r"(smem_u32(smem_dst)),
                         "l"(map),
                         "r"(c0),
                         "r"(c1),
                         "r"(c2),
                         "r"(c3),
                         "r"(smem_u32(bar))
                         : "memory");
        }
        // 4D tiled box store, shared -> global, tracked by the issuing thread's bulk groups
        __device__ __forceinline__ void
            tma_store_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3, const void* smem_src)
        {
            asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(map),
                         "r"(c0),
                         "r"(c1),
                         "r"(c2),
                         "r"(c3),
                         "r"(smem_u32(smem_src))
                         : "memory");
        }
    }

    // value representation inside the kernel: P = one 8-byte component
    template <typename T>
    struct StreamVal;
    template <>
    struct StreamVal<float>
    {
        using P                  = pk2;
        using C2                 = pk2c;
        using U                  = float4;
        static constexpr int VEC = 2; // columns per thread
        __device__ static __forceinline__ C2 unpack(const float4 v, float sgn)
        {
            C2 r;
            r.x = pk2(v.x, v.z);
            r.y = pk2(v.y * sgn, v.w * sgn);
            return r;
        }
        __device__ static __forceinline__ float4 pack(const C2 c, float sx, float sy)
        {
            return make_float4(c.x.v.x * sx, c.y.v.x * sy, c.x.v.y * sx, c.y.v.y * sy);
        }
        // c * w for a scalar twiddle w
        __device__ static __forceinline__ C2 twmul(const C2 c, const float2 w)
        {
            const float2 wx = make_float2(w.x, w.x), wy = make_float2(w.y, w.y), nwy = make_float2(-w.y, -w.y);
            C2           r;
            r.x = pk2(__ffma2_rn(c.x.v, wx, __fmul2_rn(c.y.v, nwy)));
            r.y = pk2(__ffma2_rn(c.x.v, wy, __fmul2_rn(c.y.v, wx)));
            return r;
        }
        // shared-memory copy of a twiddle: both parts already broadcast to a register pair
        using TWS = float4;
        __device__ static __forceinline__ TWS tws(const float2 w)
        {
            return make_float4(w.x, w.x, w.y, w.y);
        }
        __device__ static __forceinline__ C2 twmul(const C2 c, const float4 w)
        {
            const float2 wx = make_float2(w.x, w.y), wy = make_float2(w.z, w.w), nwy = make_float2(-w.z, -w.w);
            C2           r;
            r.x = pk2(__ffma2_rn(c.x.v, wx, __fmul2_rn(c.y.v, nwy)));
            r.y = pk2(__ffma2_rn(c.x.v, wy, __fmul2_rn(c.y.v, wx)));
            return r;
        }
    };
    template <>
    struct StreamVal<double>
    {
        using P                  = double;
        using C2                 = double2;
        using U                  = double2;
        static constexpr int VEC = 1;
        __device__ static __forceinline__ C2 unpack(const double2 v, double sgn)
        {
            return make_double2(v.x, v.y * sgn);
        }
        __device__ static __forceinline__ double2 pack(const C2 c, double sx, double sy)
        {
            return make_double2(c.x * sx, c.y * sy);
        }
        __device__ static __forceinline__ C2 twmul(const C2 c, const double2 w)
        {
            return cmul(c, w);
        }
        using TWS = double2;
        __device__ static __forceinline__ TWS tws(const double2 w)
        {
            return w;
        }
    };

    // UN = 16-byte units per tile row: 8 (128-byte rows, the width strided HBM traffic wants) or 4
    // (64-byte rows: half the shared memory, for tiles that come out of L2)
    // Single precision, one column per thread: twice the threads of the packed form for the same tile
    // (more warps to hide the latencies of each phase), ordinary scalar arithmetic, 8-byte units.
    struct StreamValScalarF
    {
        using P                  = float;
        using C2                 = float2;
        using U                  = float2;
        static constexpr int VEC = 1;
        __device__ static __forceinline__ C2 unpack(const float2 v, float sgn)
        {
            return make_float2(v.x, v.y * sgn);
        }
        __device__ static __forceinline__ float2 pack(const C2 c, float sx, float sy)
        {
            return make_float2(c.x * sx, c.y * sy);
        }
        __device__ static __forceinline__ C2 twmul(const C2 c, const float2 w)
        {
            return cmul(c, w);
        }
        using TWS = float2;
        __device__ static __forceinline__ TWS tws(const float2 w)
        {
            return w;
        }
    };
    template <typename T, bool SC>
    struct StreamValSel
    {
        using type = StreamVal<T>;
    };
    template <>
    struct StreamValSel<float, true>
    {
        using type = StreamValScalarF;
    };

    // SC: single precision in scalar form (one column per thread) instead of packed pairs
    template <class C, int UN = 8, bool SC = false>
    struct ColStream
    {
        using Cfg                        = C;
        using T                          = typename C::T;
        using SV                         = typename StreamValSel<T, SC>::type;
        using P                          = typename SV::P;
        using C2                         = typename SV::C2;
        using U                          = typename SV::U;
        static constexpr int VEC         = SV::VEC;
        static constexpr int UNITS       = UN * 16 / (int)sizeof(U); // per-thread units in a row segment of UN * 16 bytes
        static constexpr int COLS        = UNITS * VEC;
        static constexpr int THREADS     = C::TPT * UNITS;
        static constexpr int EPT         = C::N / C::TPT;
        static constexpr int BOX_ROWS    = C::N < 256 ? C::N : 256;
        static constexpr int NBOX        = C::N / BOX_ROWS;
        static constexpr unsigned ROW_BYTES   = (unsigned)UN * 16u;
        static constexpr unsigned STAGE_BYTES = (unsigned)C::N * ROW_BYTES;
        static constexpr int      XROWS       = C::N + (C::N >> 5) + 1; // one pad row per 32 keeps both passes conflict-free
        static constexpr size_t   XCHG_BYTES  = C::NPASS > 1 ? (size_t)XROWS * UNITS * sizeof(P) : 0;
        // two-pass kernels keep the twiddles of their second pass in shared memory (16 bytes per entry):
        // the L1 cache left beside ~200 KB of shared memory is too small to hold them against the
        // kernel's own store traffic
        static constexpr bool     TW_SMEM     = C::NPASS == 2;
        static constexpr int      TW_ENTRIES  = TW_SMEM ? (C::FL::get(1) - 1) * C::FL::get(0) : 0;
        static constexpr size_t   TW_BYTES    = (size_t)TW_ENTRIES * sizeof(typename SV::TWS);
        static constexpr size_t   SMEM_BYTES  = 256 + STAGE_BYTES + XCHG_BYTES + 16 + TW_BYTES; // slack to align the stage to 256 bytes
        // results leave through the exchange buffer, half a tile at a time, as tensor stores
        static constexpr int      OBOX_ROWS   = C::N / 2 < 256 ? C::N / 2 : 256;
        static constexpr int      ONBOX       = (C::N / 2) / OBOX_ROWS; // boxes per half tile
        static_assert(C::NPASS < 2 || XCHG_BYTES >= (size_t)(C::N / 2) * ROW_BYTES, "half a tile must fit the exchange buffer");
        static_assert((C::N & (C::N - 1)) == 0 && C::N >= 32, "power-of-two lengths only");
        __device__ static __forceinline__ int prow(int e)
        {
            return e + (e >> 5);
        }
    };

    template <class CC, int P, class TWP>
    __device__ __forceinline__ void colstream_compute(typename CC::C2 (&r)[CC::EPT], const TWP* __restrict__ tw, const int tl)
    {
        using C  = typename CC::Cfg;
        using PP = ColWidePass<C, P>;
        static_assert(PP::FULL && PP::BPT * PP::W == CC::EPT, "every radix must divide the points per thread");
#pragma unroll
        for(int i = 0; i < PP::BPT; ++i)
        {
            if constexpr(P > 0)
            {
                const int k = (tl + i * C::TPT) % PP::CH;
#pragma unroll
                for(int j = 1; j < PP::W; ++j)
                    r[i * PP::W + j] = CC::SV::twmul(r[i * PP::W + j], tw[(CC::TW_SMEM ? 0 : PP::TWO) + (j - 1) * PP::CH + k]);
            }
            Butterfly<PP::W, typename CC::C2>::run(*reinterpret_cast<typename CC::C2(*)[PP::W]>(&r[i * PP::W]));
        }
    }

    // exchange after pass P: results of pass P (in r) -> inputs of pass P+1 (in r), one component at a time
    template <class CC, int P>
    __device__ __forceinline__ void colstream_exchange(typename CC::C2 (&r)[CC::EPT],
                                                       typename CC::P* xs,
                                                       const int       tl,
                                                       const int       u,
                                                       const bool      first_of_tile)
    {
        using C  = typename CC::Cfg;
        using PP = ColWidePass<C, P>;
        using PN = ColWidePass<C, P + 1>;
#pragma unroll
        for(int half = 0; half < 2; ++half)
        {
            // the buffer must be free: its previous readers are past a barrier (the stage barrier
            // covers the first use in a tile)
            if(!(first_of_tile && half == 0))
                __syncthreads();
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b  = tl + i * C::TPT;
                const int k  = b % PP::CH;
                const int e0 = (b / PP::CH) * (PP::W * PP::CH) + k;
#pragma unroll
                for(int j = 0; j < PP::W; ++j)
                    xs[CC::prow(e0 + j * PP::CH) * CC::UNITS + u] = half == 0 ? r[i * PP::W + j].x : r[i * PP::W + j].y;
            }
            __syncthreads();
#pragma unroll
            for(int i = 0; i < PN::BPT; ++i)
            {
                const int b = tl + i * C::TPT;
#pragma unroll
                for(int j = 0; j < PN::W; ++j)
                {
                    const typename CC::P v = xs[CC::prow(b + j * PN::NB) * CC::UNITS + u];
                    if(half == 0)
                        r[i * PN::W + j].x = v;
                    else
                        r[i * PN::W + j].y = v;
                }
            }
        }
    }

    template <class CC, int P, bool BLK, class TWP>
    __device__ __forceinline__ void colstream_from(typename CC::C2 (&r)[CC::EPT],
                                                   typename CC::P* xs,
                                                   const TWP* __restrict__   tw,
                                                   const int                 tl,
                                                   const int                 u,
                                                   const b200fft_kargs&      a,
                                                   typename CC::Cfg::T2*     gout,
                                                   const long long           obase,
                                                   const typename CC::T      sx,
                                                   const typename CC::T      sy)
    {
        using C  = typename CC::Cfg;
        using PP = ColWidePass<C, P>;
        using T2 = typename C::T2;
        using U  = typename CC::U;
        colstream_compute<CC, P, TWP>(r, tw, tl);
        if constexpr(P == C::NPASS - 1)
        {
#pragma unroll
            for(int i = 0; i < PP::BPT; ++i)
            {
                const int b   = tl + i * C::TPT;
                const int k   = b % PP::CH;
                const int e0  = (b / PP::CH) * (PP::W * PP::CH) + k;
                T2*       q   = gout + (long long)e0 * a.out.es;
                const long long ost = (long long)PP::CH * a.out.es;
#pragma unroll
                for(int j = 0; j < PP::W; ++j)
                {
                    T2* dst = BLK ? blk_address<T2>(a.out, obase, e0 + j * PP::CH) : q + j * ost;
                    *reinterpret_cast<U*>(dst) = CC::SV::pack(r[i * PP::W + j], sx, sy);
                }
            }
        }
        else
        {
            colstream_exchange<CC, P>(r, xs, tl, u, P == 0);
            colstream_from<CC, P + 1, BLK, TWP>(r, xs, tw, tl, u, a, gout, obase, sx, sy);
        }
    }

    // all passes from P on, results of the last pass left in r
    template <class CC, int P, class TWP>
    __device__ __forceinline__ void colstream_run(typename CC::C2 (&r)[CC::EPT],
                                                  typename CC::P* xs,
                                                  const TWP* __restrict__ tw,
                                                  const int               tl,
                                                  const int               u)
    {
        using C = typename CC::Cfg;
        colstream_compute<CC, P, TWP>(r, tw, tl);
        if constexpr(P < C::NPASS - 1)
        {
            colstream_exchange<CC, P>(r, xs, tl, u, P == 0);
            colstream_run<CC, P + 1, TWP>(r, xs, tw, tl, u);
        }
    }

    // Results of the last pass (in r) -> global memory as tensor stores, half a tile at a time through the
    // exchange buffer `xs` (free once every thread is past its last exchange read).  Thread 0 calls
    // issue(first row of the box, shared-memory source) for every box and commits them as one bulk group;
    // it must have waited for the reads of the previous tile's groups before the buffer was last reused.
    template <class CC, class Issue>
    __device__ __forceinline__ void colstream_store_staged(typename CC::C2 (&r)[CC::EPT],
                                                           typename CC::P*      xs,
                                                           const int            tl,
                                                           const int            u,
                                                           const int            tid,
                                                           const typename CC::T sx,
                                                           const typename CC::T sy,
                                                           Issue&&              issue)
    {
        using C  = typename CC::Cfg;
        using U  = typename CC::U;
        using PL = ColWidePass<C, C::NPASS - 1>;
        static_assert(PL::W * PL::CH == C::N && PL::W % 2 == 0, "the last pass spans the whole transform");
        U* ost = reinterpret_cast<U*>(xs);
#pragma unroll
        for(int half = 0; half < 2; ++half)
        {
            if(half == 1 && tid == 0)
                ptx::bulk_wait_read<0>(); // the first half has been read out of the buffer
            // half 0: every thread is past its last read of the exchange buffer
            __syncthreads();
#pragma unroll
            for(int i = 0; i < PL::BPT; ++i)
            {
                const int b = tl + i * C::TPT; // < CH: output rows b + j * CH
#pragma unroll
                for(int j = half * (PL::W / 2); j < (half + 1) * (PL::W / 2); ++j)
                    ost[(b + (j - half * (PL::W / 2)) * PL::CH) * CC::UNITS + u] = CC::SV::pack(r[i * PL::W + j], sx, sy);
            }
            ptx::fence_async_smem(); // written through the generic proxy, read by the copy engine
            __syncthreads();
            if(tid == 0)
            {
#pragma unroll
                for(int bx = 0; bx < CC::ONBOX; ++bx)
                    issue(half * (C::N / 2) + bx * CC::OBOX_ROWS,
                          reinterpret_cast<const unsigned char*>(ost) + (size_t)bx * CC::OBOX_ROWS * CC::ROW_BYTES);
                ptx::bulk_commit();
            }
        }
    }

    // kargs as for the other column kernels; aux[3] = device error flag (int*).  `map` describes
    // the input array: dimension 0 = 8-byte elements along the columns, 1 = the transform,
    // 2 / 3 = the outer dimensions on[1] / on[2].
    //
    // TS: the results leave as tensor stores (the copy engine writes the strided rows; the warps do not
    // wait on 1024 scattered lines per tile): each half of the tile goes through the exchange buffer,
    // which is free after the last pass, and `omap` describes the output array like `map` the input
    // (its dimension order in bits 8-13 of iaux[3]).  Without TS the threads store from registers.
    template <class C, bool BLK, bool SC = false, bool TS = false>
    __global__ void __launch_bounds__((ColStream<C, 8, SC>::THREADS), C::MINB)
        stockham_colstream_kernel(const __grid_constant__ b200fft_kargs a,
                                  const __grid_constant__ CUtensorMap   map,
                                  const __grid_constant__ CUtensorMap   omap)
    {
        static_assert(!TS || (!BLK && C::NPASS >= 2), "tensor stores: plain output, at least two passes");
        using CC = ColStream<C, 8, SC>;
        using T  = typename C::T;
        using T2 = typename C::T2;
        using U  = typename CC::U;
        using C2 = typename CC::C2;
        extern __shared__ unsigned char smem_dyn[];
        // the stage is the destination of tensor copies: 128-byte alignment (256 to be safe)
        unsigned char* smem_raw
            = smem_dyn + ((256u - (ptx::smem_u32(smem_dyn) & 255u)) & 255u);
        U*                 stage = reinterpret_cast<U*>(smem_raw);
        typename CC::P*    xs    = reinterpret_cast<typename CC::P*>(smem_raw + CC::STAGE_BYTES);
        uint64_t*          full  = reinterpret_cast<uint64_t*>(smem_raw + CC::STAGE_BYTES + CC::XCHG_BYTES);

        const int tid = threadIdx.x;
        const int u   = tid % CC::UNITS;
        const int tl  = tid / CC::UNITS;
        const T2* __restrict__ tw = reinterpret_cast<const T2*>(a.twiddles);
        const T sgn = a.inverse ? (T)-1 : (T)1;
        const T sx  = a.use_scale ? (T)a.scale : (T)1;
        const T sy  = sx * sgn;
        int*    err = reinterpret_cast<int*>(const_cast<void*>(a.aux[3]));

        const unsigned long long ntiles = (unsigned long long)a.ntile0 * a.on[1] * a.on[2];
        const unsigned long long first  = blockIdx.x;
        const unsigned long long stride = gridDim.x;

        typename CC::SV::TWS* tws = reinterpret_cast<typename CC::SV::TWS*>(smem_raw + CC::STAGE_BYTES + CC::XCHG_BYTES + 16);
        if constexpr(CC::TW_SMEM)
            for(int i = tid; i < CC::TW_ENTRIES; i += CC::THREADS)
                tws[i] = CC::SV::tws(tw[C::FL::tw_offset(1) + i]);
        if(tid == 0)
        {
            ptx::mbar_init(full, 1);
            ptx::fence_mbar_init();
        }
        __syncthreads();

        // thread 0 only: the boxes of one tile.  The tensor map lists its dimensions 1..3 by ascending
        // stride; iaux[3] tells where the transform (bits 0-1), outer 1 (2-3) and outer 2 (4-5) ended up.
        const int pe = (int)(a.iaux[3] & 3), p1 = (int)((a.iaux[3] >> 2) & 3), p2 = (int)((a.iaux[3] >> 4) & 3);
        auto issue_load = [&](unsigned long long tile) {
            const TilePos tp = decode_tile(a, (unsigned)tile, CC::COLS);
            ptx::mbar_expect_tx(full, CC::STAGE_BYTES + B200FFT_TEST_EXTRA_TX);
#pragma unroll
            for(int bx = 0; bx < CC::NBOX; ++bx)
            {
                const int row = bx * CC::BOX_ROWS;
                const int c1  = pe == 0 ? row : (p1 == 0 ? (int)tp.i1 : (int)tp.i2);
                const int c2  = pe == 1 ? row : (p1 == 1 ? (int)tp.i1 : (int)tp.i2);
                const int c3  = pe == 2 ? row : (p1 == 2 ? (int)tp.i1 : (int)tp.i2);
                ptx::tma_load_4d(reinterpret_cast<unsigned char*>(stage) + (size_t)bx * CC::BOX_ROWS * CC::ROW_BYTES,
                                 &map,
                                 (int)(tp.i0_first * (unsigned)(sizeof(T2) / 8)),
                                 c1,
                                 c2,
                                 c3,
                                 full);
            }
        };
        if(tid == 0 && first < ntiles)
            issue_load(first);

        unsigned phase = 0;
        for(unsigned long long tile = first; tile < ntiles; tile += stride)
        {
            const bool landed = ptx::mbar_wait(full, phase);
            phase ^= 1u;
            if constexpr(TS)
                if(tid == 0)
                    ptx::bulk_wait_read<0>(); // the previous tile's stores have read the exchange buffer
            C2 r[CC::EPT];
            if(landed)
            {
                // pass-0 inputs: butterfly tl reads rows tl + j * NB0
                using P0 = ColWidePass<C, 0>;
                static_assert(P0::BPT * P0::W == CC::EPT && P0::FULL, "pass 0 must cover the points of a thread");
#pragma unroll
                for(int i = 0; i < P0::BPT; ++i)
#pragma unroll
                    for(int j = 0; j < P0::W; ++j)
                        r[i * P0::W + j] = CC::SV::unpack(stage[(tl + i * C::TPT + j * P0::NB) * CC::UNITS + u], sgn);
            }
            // the stage is free once every thread has taken its points; a wait that gave up is
            // learnt by the whole CTA here
            if(__syncthreads_or(landed ? 0 : 1))
            {
                if(tid == 0)
                {
                    if(err)
                        atomicExch(err, 1);
                    ptx::mbar_wait(full, phase ^ 1u); // the copy may still be in flight: give it one more bounded wait
                    if constexpr(TS)
                        ptx::bulk_wait_all(); // our own stores
                }
                __syncthreads();
                return;
            }
            const unsigned long long next = tile + stride;
            if(tid == 0 && next < ntiles)
                issue_load(next);

            const TilePos   tp    = decode_tile(a, (unsigned)tile, CC::COLS);
            if constexpr(TS)
            {
                if constexpr(CC::TW_SMEM)
                    colstream_run<CC, 0>(r, xs, tws, tl, u);
                else
                    colstream_run<CC, 0>(r, xs, tw, tl, u);
                const int oe = (int)((a.iaux[3] >> 8) & 3), o1 = (int)((a.iaux[3] >> 10) & 3);
                colstream_store_staged<CC>(r, xs, tl, u, tid, sx, sy, [&](int row, const unsigned char* src) {
                    const int c1 = oe == 0 ? row : (o1 == 0 ? (int)tp.i1 : (int)tp.i2);
                    const int c2 = oe == 1 ? row : (o1 == 1 ? (int)tp.i1 : (int)tp.i2);
                    const int c3 = oe == 2 ? row : (o1 == 2 ? (int)tp.i1 : (int)tp.i2);
                    ptx::tma_store_4d(&omap, (int)(tp.i0_first * (unsigned)(sizeof(T2) / 8)), c1, c2, c3, src);
                });
            }
            else
            {
                const long long obase = view_base(a.out, tp.i0_first + u * CC::VEC, tp.i1, tp.i2);
                T2*             gout  = reinterpret_cast<T2*>(a.out.p[0]) + obase;
                if constexpr(CC::TW_SMEM)
                    colstream_from<CC, 0, BLK>(r, xs, tws, tl, u, a, gout, obase, sx, sy);
                else
                    colstream_from<CC, 0, BLK>(r, xs, tw, tl, u, a, gout, obase, sx, sy);
            }
        }
        if constexpr(TS)
            if(tid == 0)
                ptx::bulk_wait_all(); // nothing of ours may be in flight when the CTA retires
    }

    // cuTensorMapEncodeTiled through the runtime's driver entry point lookup (the library does not link libcuda)
    typedef CUresult (*tmap_encode_fn)(CUtensorMap*,
                                       CUtensorMapDataType,
                                       cuuint32_t,
                                       void*,
                                       const cuuint64_t*,
                                       const cuuint64_t*,
                                       const cuuint32_t*,
                                       const cuuint32_t*,
                                       CUtensorMapInterleave,
                                       CUtensorMapSwizzle,
                                       CUtensorMapL2promotion,
                                       CUtensorMapFloatOOBfill);
    inline tmap_encode_fn tmap_encoder()
    {
        static tmap_encode_fn  fn = nullptr;
        static std::once_flag once;
        std::call_once(once, [] {
            void*                           p = nullptr;
            cudaDriverEntryPointQueryResult q;
            if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess
               && q == cudaDriverEntryPointSuccess)
                fn = reinterpret_cast<tmap_encode_fn>(p);
        });
        return fn;
    }

    // One side of a column stage as a 4D tensor of 8-byte elements: dimension 0 runs along the columns;
    // the transform dimension and the two outer dimensions follow by ascending stride (unit-length
    // dimensions last, with a stride that continues the sequence).  `perm` tells the kernel where the
    // transform (bits 0-1), outer 1 (2-3) and outer 2 (4-5) ended up.  False: the view does not fit a map.
    inline bool colstream_tile_map(CUtensorMap*          map,
                                   long long*            perm_out,
                                   const b200fft_ioview& v,
                                   const b200fft_kargs&  a,
                                   unsigned              n,
                                   size_t                elem_bytes,
                                   unsigned              box_rows)
    {
        tmap_encode_fn enc = tmap_encoder();
        if(!enc)
            return false;
        if(v.es <= 0 || (a.on[1] > 1 && v.os[1] <= 0) || (a.on[2] > 1 && v.os[2] <= 0))
            return false;
        struct Dim
        {
            cuuint64_t len, stride;
            int        which; // 0 transform, 1 outer 1, 2 outer 2
        };
        Dim d[3] = {{(cuuint64_t)n, (cuuint64_t)v.es * elem_bytes, 0},
                    {a.on[1], (cuuint64_t)v.os[1] * elem_bytes, 1},
                    {a.on[2], (cuuint64_t)v.os[2] * elem_bytes, 2}};
        auto before = [](const Dim& x, const Dim& y) {
            const bool ux = x.len <= 1 && x.which != 0, uy = y.len <= 1 && y.which != 0;
            if(ux != uy)
                return uy; // real dimensions first
            return x.stride < y.stride;
        };
        for(int i = 0; i < 3; ++i)
            for(int j = i + 1; j < 3; ++j)
                if(before(d[j], d[i]))
                    std::swap(d[i], d[j]);
        for(int i = 1; i < 3; ++i)
            if(d[i].len <= 1 && d[i].which != 0)
            {
                d[i].len    = 1;
                d[i].stride = d[i - 1].stride * d[i - 1].len;
            }
        for(int i = 0; i < 3; ++i)
            if(d[i].stride >= (1ull << 40) || d[i].stride % 16)
                return false;
        const cuuint64_t ce         = elem_bytes / 8;
        const cuuint64_t dims[4]    = {(cuuint64_t)a.on[0] * ce, d[0].len, d[1].len, d[2].len};
        const cuuint64_t strides[3] = {d[0].stride, d[1].stride, d[2].stride};
        cuuint32_t       box[4]     = {16, 1, 1, 1};
        long long        perm       = 0;
        for(int i = 0; i < 3; ++i)
        {
            if(d[i].which == 0)
                box[1 + i] = (cuuint32_t)box_rows;
            perm |= (long long)i << (2 * d[i].which);
        }
        *perm_out                = perm;
        const cuuint32_t estr[4] = {1, 1, 1, 1};
        return enc(map,
                   CU_TENSOR_MAP_DATA_TYPE_UINT64,
                   4,
                   v.p[0],
                   dims,
                   strides,
                   box,
                   estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
               == CUDA_SUCCESS;
    }

    template <class C, bool BLK, bool SC, bool TS>
    cudaError_t colstream_grid(int dev, unsigned long long* grid)
    {
        using CC = ColStream<C, 8, SC>;
        static int        blocks_per_sm[64] = {};
        static int        sm_count[64]      = {};
        static std::mutex mtx;
        auto              kern = stockham_colstream_kernel<C, BLK, SC, TS>;
        std::lock_guard<std::mutex> g(mtx);
        if(!blocks_per_sm[dev])
        {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CC::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            int nb = 0;
            e      = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kern, CC::THREADS, CC::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
            blocks_per_sm[dev] = nb > 0 ? nb : 1;
        }
        *grid = (unsigned long long)blocks_per_sm[dev] * sm_count[dev];
        return cudaSuccess;
    }

    template <class C, bool BLK, bool SC = false>
    cudaError_t launch_colstream_kernel(const b200fft_kargs& a, unsigned long long ntiles, cudaStream_t stream)
    {
        using CC = ColStream<C, 8, SC>;
        using T2 = typename C::T2;
        int dev  = 0;
        cudaGetDevice(&dev);
        if(dev < 0 || dev >= 64)
            return cudaErrorInvalidDevice;
        // plain output that a tensor map can describe leaves through tensor stores (B200FFT_COLTMA_REG_STORES,
        // read once, keeps the stores in the threads: measurements)
        static const bool reg_stores = getenv("B200FFT_COLTMA_REG_STORES") != nullptr;
        constexpr bool    CAN_TS     = !BLK && C::NPASS >= 2;
        if(ntiles == 0)
            return cudaSuccess;
        if(ntiles > 0x7fffffffull)
            return cudaErrorInvalidConfiguration;
        if(!tmap_encoder())
            return cudaErrorNotSupported;
        alignas(64) CUtensorMap map, omap;
        long long               perm = 0, operm = 0;
        if(!colstream_tile_map(&map, &perm, a.in, a, (unsigned)C::N, sizeof(T2), (unsigned)CC::BOX_ROWS))
            return cudaErrorInvalidValue;
        bool ts = false;
        // (bit 32 of iaux[3], set by the planner: the output is another GPU's memory, keep to plain stores)
        if constexpr(CAN_TS)
            ts = !reg_stores && !(a.iaux[3] & (1ll << 32)) && (reinterpret_cast<size_t>(a.out.p[0]) % 16 == 0)
                 && colstream_tile_map(&omap, &operm, a.out, a, (unsigned)C::N, sizeof(T2), (unsigned)CC::OBOX_ROWS);
        if(!ts)
            omap = map;
        b200fft_kargs ka = a;
        ka.iaux[3]       = perm | (operm << 8);
        unsigned long long grid = 0;
        if constexpr(CAN_TS)
            if(ts)
            {
                cudaError_t e = colstream_grid<C, BLK, SC, true>(dev, &grid);
                if(e != cudaSuccess)
                    return e;
                if(grid > ntiles)
                    grid = ntiles;
                stockham_colstream_kernel<C, BLK, SC, true><<<(unsigned)grid, CC::THREADS, CC::SMEM_BYTES, stream>>>(ka, map, omap);
                return cudaGetLastError();
            }
        cudaError_t e = colstream_grid<C, BLK, SC, false>(dev, &grid);
        if(e != cudaSuccess)
            return e;
        if(grid > ntiles)
            grid = ntiles;
        stockham_colstream_kernel<C, BLK, SC, false><<<(unsigned)grid, CC::THREADS, CC::SMEM_BYTES, stream>>>(ka, map, omap);
        return cudaGetLastError();
    }
} // namespace b200fft
