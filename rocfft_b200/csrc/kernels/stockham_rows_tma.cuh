// Persistent, TMA-pipelined Stockham kernel for contiguous batches of rows.
//
// Role in the reference: the same single-kernel Stockham scheme as
// stockham_engine.cuh (library/src/device/generator/stockham_gen_rr.h), for the
// case the benchmark configurations hit most: unit-stride transforms stored
// back to back.  The reference relies on many resident workgroups to hide HBM
// latency; on B200 that leaves the memory system idle whenever the resident
// CTAs happen to compute at the same time.  Here each CTA is persistent and
// moves its tiles with the bulk-copy engine instead:
//
//   cp.async.bulk global -> shared (complete_tx on an mbarrier), NST stages deep,
//   radix passes in shared memory,
//   cp.async.bulk shared -> global for the result,
//
// so loads of the next tiles and the store of the previous tile are in
// flight while the threads compute, and no thread ever waits on a global load.
// Three modes share the pipeline:
//   MODE_C2C  complex rows of N points in, N points out (in place or not);
//   MODE_R2C  rows of 2N reals (read as N complex) in, N+1 Hermitian points out:
//             even-length real forward transform with its post-processing done
//             in shared memory (reference: rtc_realcomplex_gen.cpp:467-557);
//   MODE_C2R  the inverse: N+1 Hermitian points in, 2N reals out.
//
// A tile is TPB consecutive rows, i.e. one contiguous range of global memory;
// a ragged last tile whose byte count is not a multiple of 16 is moved with
// plain loads and stores.  Base pointers must be 16-byte aligned (the launch
// layer checks and otherwise uses the non-TMA kernel).  Every mbarrier wait is
// bounded: on expiry the whole CTA learns of it at the next barrier, raises the
// plan's device error flag, drains its own bulk stores, gives the loads still in
// flight one more bounded wait and returns.  No multicast, no clusters: the kernel is legal
// in multi-GPU runs.
#pragma once
#include "stockham_engine.cuh"
#include <cstdint>
#include <mutex>

namespace b200fft
{
    enum RowsMode
    {
        MODE_C2C = 0,
        MODE_R2C = 1,
        MODE_C2R = 2,
    };

#ifndef B200FFT_MBAR_SPIN
#define B200FFT_MBAR_SPIN (1u << 22) // try_wait attempts before a wait gives up
#endif
// Test hook: bytes added to every expected transaction count.  With a non-zero value no load
// phase ever completes, so the bounded waits run out although every copy has landed; the
// wait-expiry test builds a probe with this and a short B200FFT_MBAR_SPIN.  Always 0 in the library.
#ifndef B200FFT_TEST_EXTRA_TX
#define B200FFT_TEST_EXTRA_TX 0u
#endif

    namespace ptx
    {
        __device__ __forceinline__ uint32_t smem_u32(const void* p)
        {
            return (uint32_t)__cvta_generic_to_shared(p);
        }
        __device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count)
        {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
        }
        __device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes)
        {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                         : "memory");
        }
        __device__ __forceinline__ void mbar_arrive(uint64_t* bar)
        {
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
        }
        __device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity)
        {
            uint32_t ok;
            asm volatile("{\n\t.reg .pred p;\n\t"
                         "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                         "selp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok)
                         : "r"(smem_u32(bar)), "r"(parity)
                         : "memory");
            return ok != 0;
        }
        // bounded wait; false on expiry
        __device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity)
        {
            for(unsigned i = 0; i < B200FFT_MBAR_SPIN; ++i)
                if(mbar_try_wait(bar, parity))
                    return true;
            return false;
        }
        __device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, unsigned bytes, uint64_t* bar)
        {
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             smem_u32(smem_dst)),
                         "l"(gsrc),
                         "r"(bytes),
                         "r"(smem_u32(bar))
                         : "memory");
        }
        __device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, unsigned bytes)
        {
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
                         "r"(smem_u32(smem_src)),
                         "r"(bytes)
                         : "memory");
        }
        __device__ __forceinline__ void bulk_commit()
        {
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        template <int N>
        __device__ __forceinline__ void bulk_wait_read()
        {
            asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
        }
        __device__ __forceinline__ void bulk_wait_all()
        {
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        }
        __device__ __forceinline__ void fence_async_smem()
        {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __device__ __forceinline__ void fence_mbar_init()
        {
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }

    // Packed single precision (KCfg with T = pk2): a "transform" of the tile is a PAIR of adjacent rows
    // whose values travel as pk2c (real parts of both rows in one register pair, imaginary parts in
    // another): every shared-memory access of the passes moves 16 bytes for two rows and every butterfly
    // instruction is a packed one, which halves the instruction count per point of these issue-bound
    // kernels.  The stages hold the rows exactly as they lie in global memory (RAW = ordinary complex).
    template <class C, int MODE, int NST>
    struct RowsTma
    {
        using T2  = typename C::T2;
        using RAW = typename C::TW2; // element type of global memory and of the stages
        static constexpr int RPT     = sizeof(T2) / sizeof(RAW); // rows per transform slot: 2 when packed
        static constexpr int TROWS   = C::TPB * RPT; // rows per tile
        static constexpr int IN_ROW  = (MODE == MODE_C2R) ? C::N + 1 : C::N;
        static constexpr int OUT_ROW = (MODE == MODE_R2C) ? C::N + 1 : C::N;
        static constexpr int ROWMAX  = IN_ROW > OUT_ROW ? IN_ROW : OUT_ROW;
        // stage size in elements, kept a multiple of 16 bytes
        static constexpr int    STAGE_ELEMS = ((TROWS * ROWMAX * (int)sizeof(RAW) + 15) / 16) * 16 / (int)sizeof(RAW);
        static constexpr size_t STAGE_BYTES = (size_t)STAGE_ELEMS * sizeof(RAW);
        static constexpr size_t WORK_BYTES  = ((sizeof(T2) * (size_t)C::SMEM_ELEMS + 15) / 16) * 16;
        static constexpr size_t SMEM_BYTES  = NST * STAGE_BYTES + WORK_BYTES + 8 * NST;
    };

    // stage <-> value conversions: one row, or two rows packed
    template <typename T2, typename RAW>
    struct RowIo
    {
        // value of slot c, point e, from rows stored with pitch `row` (rows at or beyond nvalid read as zero)
        __device__ static __forceinline__ T2 load(const RAW* stage, int c, int e, int row, unsigned nvalid)
        {
            T2 v;
            v.x = 0;
            v.y = 0;
            if((unsigned)c < nvalid)
                v = stage[c * row + e];
            return v;
        }
        __device__ static __forceinline__ void store(RAW* stage, int c, int e, int row, const T2 v)
        {
            stage[c * row + e] = v;
        }
        template <typename S>
        __device__ static __forceinline__ decltype(T2::x) bcast(S s)
        {
            return (decltype(T2::x))s;
        }
    };
    template <>
    struct RowIo<pk2c, float2>
    {
        __device__ static __forceinline__ pk2c load(const float2* stage, int c, int e, int row, unsigned nvalid)
        {
            float2 a = make_float2(0.f, 0.f), b = make_float2(0.f, 0.f);
            if((unsigned)(2 * c) < nvalid)
                a = stage[(2 * c) * row + e];
            if((unsigned)(2 * c + 1) < nvalid)
                b = stage[(2 * c + 1) * row + e];
            pk2c v;
            v.x = pk2(a.x, b.x);
            v.y = pk2(a.y, b.y);
            return v;
        }
        __device__ static __forceinline__ void store(float2* stage, int c, int e, int row, const pk2c v)
        {
            stage[(2 * c) * row + e]     = make_float2(v.x.v.x, v.y.v.x);
            stage[(2 * c + 1) * row + e] = make_float2(v.x.v.y, v.y.v.y);
        }
        template <typename S>
        __device__ static __forceinline__ pk2 bcast(S s)
        {
            return pk2((float)s, (float)s);
        }
    };

    // kargs: in.p[0] / out.p[0] 16-byte aligned bases, on[0] = number of rows,
    // ntile0 = number of tiles, aux[0] = half-length twiddles (real modes),
    // aux[3] = device error flag (int*).
    template <class C, int MODE, int NST>
    __global__ void __launch_bounds__(C::THREADS, C::MINB)
        stockham_rows_tma_kernel(const __grid_constant__ b200fft_kargs a)
    {
        using T   = typename C::T;
        using T2  = typename C::T2;
        using R   = RowsTma<C, MODE, NST>;
        using RAW = typename R::RAW;
        using IO  = RowIo<T2, RAW>;
        static_assert(!C::COL, "row layout only");
        static_assert(C::NPASS >= 2, "needs at least two passes");
        extern __shared__ __align__(128) unsigned char smem_raw[];
        RAW*      stages = reinterpret_cast<RAW*>(smem_raw);
        T2*       sm     = reinterpret_cast<T2*>(smem_raw + NST * R::STAGE_BYTES);
        uint64_t* full   = reinterpret_cast<uint64_t*>(smem_raw + NST * R::STAGE_BYTES + R::WORK_BYTES);

        const int      tid     = threadIdx.x;
        const int      c       = tid / C::TPT;
        const int      t       = tid % C::TPT;
        const bool     inverse = (MODE == MODE_C2C) && a.inverse != 0;
        const bool     use_sc  = a.use_scale != 0;
        const T        scale   = IO::bcast(a.scale);
        const unsigned nrows   = a.on[0];
        const unsigned ntiles  = a.ntile0;
        const RAW* __restrict__ tw  = reinterpret_cast<const RAW*>(a.twiddles);
        const RAW* __restrict__ htw = reinterpret_cast<const RAW*>(a.aux[0]);
        int*           err          = reinterpret_cast<int*>(const_cast<void*>(a.aux[3]));
        const RAW*     gin          = reinterpret_cast<const RAW*>(a.in.p[0]);
        RAW*           gout         = reinterpret_cast<RAW*>(a.out.p[0]);

        const unsigned first   = blockIdx.x;
        const unsigned stride  = gridDim.x;
        const unsigned mycount = ntiles > first ? (ntiles - first + stride - 1) / stride : 0;

        if(tid == 0)
        {
            for(int s = 0; s < NST; ++s)
                ptx::mbar_init(&full[s], 1);
            ptx::fence_mbar_init();
        }
        __syncthreads();

        auto tile_rows = [&](unsigned k) -> unsigned {
            const unsigned tile = first + k * stride;
            return min((unsigned)R::TROWS, nrows - tile * (unsigned)R::TROWS);
        };
        // thread 0 only
        auto issue_load = [&](unsigned k) {
            const unsigned tile  = first + k * stride;
            const unsigned bytes = tile_rows(k) * (unsigned)(R::IN_ROW * sizeof(RAW));
            const int      s     = (int)(k % NST);
            if((bytes & 15u) == 0)
            {
                ptx::mbar_expect_tx(&full[s], bytes + B200FFT_TEST_EXTRA_TX);
                ptx::bulk_load(stages + (size_t)s * R::STAGE_ELEMS,
                               gin + (size_t)tile * R::TROWS * R::IN_ROW,
                               bytes,
                               &full[s]);
            }
            else
                ptx::mbar_arrive(&full[s]); // ragged tile: moved by the threads when it is consumed
        };

        if(tid == 0)
            for(unsigned k = 0; k + 1 < (unsigned)NST && k < mycount; ++k)
                issue_load(k);

        for(unsigned k = 0; k < mycount; ++k)
        {
            const int      s      = (int)(k % NST);
            const unsigned tile   = first + k * stride;
            const unsigned nvalid = tile_rows(k); // rows
            RAW*           stage  = stages + (size_t)s * R::STAGE_ELEMS;
            // a wait that gave up is learnt by the whole CTA at this barrier, so that it leaves in step
            const bool landed = ptx::mbar_wait(&full[s], (k / NST) & 1u);
            if(__syncthreads_or(landed ? 0 : 1))
            {
                if(tid == 0)
                {
                    if(err)
                        atomicExch(err, 1);
                    ptx::bulk_wait_all(); // our own stores
                    // loads issued for later tiles may still be in flight towards this CTA's shared
                    // memory: give each one more bounded wait before the memory is released
                    for(unsigned kk = k; kk < k + (unsigned)NST - 1 && kk < mycount; ++kk)
                        ptx::mbar_wait(&full[kk % NST], (kk / NST) & 1u);
                }
                __syncthreads();
                return;
            }
            const unsigned in_bytes  = nvalid * (unsigned)(R::IN_ROW * sizeof(RAW));
            const unsigned out_bytes = nvalid * (unsigned)(R::OUT_ROW * sizeof(RAW));
            if(in_bytes & 15u)
            {
                const RAW* src = gin + (size_t)tile * R::TROWS * R::IN_ROW;
                for(unsigned i = tid; i < nvalid * R::IN_ROW; i += C::THREADS)
                    stage[i] = src[i];
                __syncthreads();
            }

            // ---------------- transform the tile ----------------
            if constexpr(MODE == MODE_C2R)
            {
                // Hermitian pre-processing: stage (N+1 points per row) -> work tile, parts exchanged
                constexpr int H     = C::N;
                constexpr int NP    = H / 2 + 1;
                constexpr int ITEMS = NP * C::TPB;
#pragma unroll 4
                for(int idx = tid; idx < ITEMS; idx += C::THREADS)
                {
                    const int cc = idx / NP;
                    const int p  = idx % NP;
                    const int q  = H - p;
                    T2        xa = IO::load(stage, cc, p, R::IN_ROW, nvalid);
                    T2        xb = IO::load(stage, cc, q, R::IN_ROW, nvalid);
                    if(p == 0)
                    {
                        xa.y = IO::bcast(0);
                        xb.y = IO::bcast(0);
                    }
                    xb.y        = -xb.y;
                    const RAW w = htw[p];
                    T2        e, d, tt;
                    e.x  = xa.x + xb.x;
                    e.y  = xa.y + xb.y;
                    d.x  = xa.x - xb.x;
                    d.y  = xa.y - xb.y;
                    tt.x = IO::bcast(w.y);
                    tt.y = IO::bcast(w.x);
                    const T2 td = cmul(tt, d);
                    T2       zp, zq;
                    zp.x = e.x + td.x;
                    zp.y = e.y + td.y;
                    zq.x = e.x - td.x;
                    zq.y = -(e.y - td.y);
                    sm[C::sidx(cc, p)] = cswap(zp);
                    if(p != q && p != 0)
                        sm[C::sidx(cc, q)] = cswap(zq);
                }
                __syncthreads();
                auto s_src = [=](int e) -> T2 { return sm[C::sidx(c, e)]; };
                auto o_dst = [=](int e, T2 v) {
                    v = cswap(v);
                    if(use_sc)
                    {
                        v.x *= scale;
                        v.y *= scale;
                    }
                    IO::store(stage, c, e, R::OUT_ROW, v);
                };
                run_passes<C, 0, true, false>(t, c, sm, tw, s_src, o_dst);
            }
            else
            {
                auto i_src = [=](int e) -> T2 {
                    const T2 v = IO::load(stage, c, e, R::IN_ROW, nvalid);
                    return inverse ? cswap(v) : v;
                };
                if constexpr(MODE == MODE_C2C)
                {
                    auto o_dst = [=](int e, T2 v) {
                        if(inverse)
                            v = cswap(v);
                        if(use_sc)
                        {
                            v.x *= scale;
                            v.y *= scale;
                        }
                        IO::store(stage, c, e, R::OUT_ROW, v);
                    };
                    run_passes<C, 0, false, false>(t, c, sm, tw, i_src, o_dst);
                }
                else
                {
                    auto s_dst = [=](int e, T2 v) { sm[C::sidx(c, e)] = v; };
                    run_passes<C, 0, false, true>(t, c, sm, tw, i_src, s_dst);
                    // Hermitian post-processing: work tile -> stage (N+1 points per row)
                    constexpr int H     = C::N;
                    constexpr int NP    = H / 2 + 1;
                    constexpr int ITEMS = NP * C::TPB;
                    const T       sc    = use_sc ? scale : IO::bcast(1);
                    const T       half  = IO::bcast(0.5);
                    // p = 0 needs no special case: with Z_H read as Z_0 the general formula gives
                    // X_0 = Re Z_0 + Im Z_0 and X_H = Re Z_0 - Im Z_0 with zero imaginary parts
#pragma unroll 4
                    for(int idx = tid; idx < ITEMS; idx += C::THREADS)
                    {
                        const int cc = idx / NP;
                        const int p  = idx % NP;
                        const int q  = H - p;
                        const T2 za = sm[C::sidx(cc, p)];
                        T2       zb = sm[C::sidx(cc, p == 0 ? 0 : q)];
                        zb.y        = -zb.y;
                        const RAW w = htw[p];
                        T2        e, d, tt;
                        e.x  = (za.x + zb.x) * half;
                        e.y  = (za.y + zb.y) * half;
                        d.x  = (za.x - zb.x) * half;
                        d.y  = (za.y - zb.y) * half;
                        tt.x = IO::bcast(w.y);
                        tt.y = IO::bcast(-w.x);
                        const T2 td = cmul(tt, d);
                        T2       xp, xq;
                        xp.x = (e.x + td.x) * sc;
                        xp.y = (e.y + td.y) * sc;
                        xq.x = (e.x - td.x) * sc;
                        xq.y = -(e.y - td.y) * sc;
                        IO::store(stage, cc, p, R::OUT_ROW, xp);
                        if(p != q)
                            IO::store(stage, cc, q, R::OUT_ROW, xq);
                    }
                }
            }

            // ---------------- hand the result to the copy engine ----------------
            ptx::fence_async_smem();
            __syncthreads();
            RAW* dst = gout + (size_t)tile * R::TROWS * R::OUT_ROW;
            if((out_bytes & 15u) == 0)
            {
                if(tid == 0)
                {
                    ptx::bulk_store(dst, stage, out_bytes);
                    ptx::bulk_commit();
                }
            }
            else
            {
                for(unsigned i = tid; i < nvalid * R::OUT_ROW; i += C::THREADS)
                    dst[i] = stage[i];
                if(tid == 0)
                    ptx::bulk_commit(); // empty group keeps the group count in step
            }
            if(tid == 0)
            {
                // the store issued one iteration ago has finished reading its stage: refill it
                ptx::bulk_wait_read<1>();
                if(k + NST - 1 < mycount)
                    issue_load(k + NST - 1);
            }
        }
        if(tid == 0)
            ptx::bulk_wait_all();
    }

    template <class C, int MODE, int NST>
    cudaError_t launch_rows_tma_kernel(const b200fft_kargs& a, unsigned long long ntiles, cudaStream_t stream)
    {
        using R                     = RowsTma<C, MODE, NST>;
        static int        blocks_per_sm[64] = {};
        static int        sm_count[64]      = {};
        static std::mutex mtx;
        int               dev = 0;
        cudaGetDevice(&dev);
        if(dev < 0 || dev >= 64)
            return cudaErrorInvalidDevice;
        auto kern = stockham_rows_tma_kernel<C, MODE, NST>;
        std::unique_lock<std::mutex> guard(mtx);
        if(!blocks_per_sm[dev])
        {
            cudaError_t e
                = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)R::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            int nb = 0;
            e      = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kern, C::THREADS, R::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
            blocks_per_sm[dev] = nb > 0 ? nb : 1;
        }
        const unsigned long long resident = (unsigned long long)blocks_per_sm[dev] * sm_count[dev];
        guard.unlock();
        if(ntiles == 0)
            return cudaSuccess;
        if(ntiles > 0x7fffffffull)
            return cudaErrorInvalidConfiguration;
        unsigned long long grid = resident;
        if(a.iaux[1] > 0 && grid > (unsigned long long)a.iaux[1])
            grid = (unsigned long long)a.iaux[1]; // the planner wants room left for a concurrent kernel
        if(grid > ntiles)
            grid = ntiles;
        kern<<<(unsigned)grid, C::THREADS, R::SMEM_BYTES, stream>>>(a);
        return cudaGetLastError();
    }
} // namespace b200fft
