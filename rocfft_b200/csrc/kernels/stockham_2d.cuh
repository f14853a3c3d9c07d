// Small two-dimensional transforms in one kernel: a CTA loads a whole N0 x N1
// image, transforms its rows, then its columns, and stores it — one HBM round
// trip instead of the two of a row pass followed by a column pass.
//
// Role in the reference: CS_KERNEL_2D_SINGLE
// (library/src/device/kernel-generator.py:693-839, tree_node_2D.cpp "Single2D").
//
// Structure.  C0 is the row configuration (length N0, one "transform per
// block" slot for each of the N1 rows), C1 the column configuration (length
// N1, N0 columns).  Both use the same number of points per thread, so both
// phases use every thread of the CTA:
//   phase 1  rows: global -> registers -> radix passes through the row-layout
//            shared tile -> the last pass leaves the row spectra in that tile;
//   phase 2  columns: the first pass reads the tile with the threads walking
//            along a row (conflict-free), middle passes exchange through a second
//            column-layout tile, the last pass stores registers -> global with
//            consecutive threads on consecutive points of dimension 0.
// Global access is the general kind (run-time strides, interleaved or planar),
// so the kernel serves any layout; in place is safe because a CTA reads its
// whole image before it writes.
//
// kargs: in.es / out.es = stride of dimension 0, in.bs / out.bs = stride of
// dimension 1, on[] / os[] = up to three outer dimensions (batch and higher FFT
// dimensions), twiddles = stacked table of the rows, aux[1] = of the columns.
#pragma once
#include "stockham_engine.cuh"

namespace b200fft
{
    template <class C0, class C1>
    struct Fused2D
    {
        using T2                         = typename C0::T2;
        static constexpr int    N0       = C0::N;
        static constexpr int    N1       = C1::N;
        static constexpr int    THREADS  = C0::THREADS;
        static constexpr int    IMG      = C0::NPAD * N1; // row-layout tile, always needed
        static constexpr int    XCHG     = C1::NPASS > 1 ? N1 * N0 : 0; // column-layout exchange tile
        static constexpr size_t SMEM_BYTES = sizeof(T2) * (size_t)(IMG + XCHG);
        static_assert(C0::TPB == N1 && C1::TPB == N0, "each configuration holds the whole image");
        static_assert(!C0::COL && C1::COL, "rows first, then columns");
        static_assert(C0::THREADS == C1::THREADS, "both phases must use the same threads");
        static_assert(C0::IOKI == IO_GENERIC && C1::IOKO == IO_GENERIC, "general global access");
    };

    template <class C0, class C1, int MINB>
    __global__ void __launch_bounds__(C0::THREADS, MINB) stockham_2d_kernel(const __grid_constant__ b200fft_kargs a)
    {
        using F  = Fused2D<C0, C1>;
        using T  = typename C0::T;
        using T2 = typename C0::T2;
        extern __shared__ __align__(16) unsigned char smem_raw[];
        T2* sm0 = reinterpret_cast<T2*>(smem_raw);
        T2* sm1 = sm0 + F::IMG;

        const int  tid     = threadIdx.x;
        const bool inverse = a.inverse != 0;
        const bool use_sc  = a.use_scale != 0;
        const T    scale   = (T)a.scale;
        const T2* __restrict__ tw0 = reinterpret_cast<const T2*>(a.twiddles);
        const T2* __restrict__ tw1 = reinterpret_cast<const T2*>(a.aux[1]);

        // which image
        const unsigned  i0    = blockIdx.x % a.on[0];
        const unsigned  r     = blockIdx.x / a.on[0];
        const long long ibase = view_base(a.in, i0, r % a.on[1], r / a.on[1]);
        const long long obase = view_base(a.out, i0, r % a.on[1], r / a.on[1]);

        // ---- rows ----
        {
            const int       c    = tid / C0::TPT; // row
            const int       t    = tid % C0::TPT;
            const long long base = ibase + (long long)c * a.in.bs;
            auto src = [&](int e) -> T2 { return gload<C0>(a.in, base, e, inverse); };
            auto dst = [=](int e, T2 v) { sm0[C0::sidx(c, e)] = v; };
            run_passes<C0, 0, false, true>(t, c, sm0, tw0, src, dst);
        }
        // ---- columns ----
        {
            const int      c  = tid % C1::TPB; // point of dimension 0
            const int      t  = tid / C1::TPB;
            b200fft_ioview vo = a.out;
            vo.es             = a.out.bs; // walk dimension 1
            const long long base = obase + (long long)c * a.out.es;
            auto src = [=](int e) -> T2 { return sm0[C0::sidx(e, c)]; };
            auto dst = [&](int e, T2 v) { gstore<C1>(vo, base, e, v, inverse, use_sc, scale); };
            run_passes<C1, 0, false, false>(t, c, sm1, tw1, src, dst);
        }
    }

    template <class C0, class C1, int MINB>
    cudaError_t launch_2d_kernel(const b200fft_kargs& a, unsigned long long nimages, cudaStream_t stream)
    {
        using F                   = Fused2D<C0, C1>;
        static std::atomic<bool> attr_done[64]; // zero-initialised; host threads may launch the same kernel concurrently
        int         dev           = 0;
        cudaGetDevice(&dev);
        auto kern = stockham_2d_kernel<C0, C1, MINB>;
        if(F::SMEM_BYTES > 48 * 1024 && dev < 64 && !attr_done[dev])
        {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            attr_done[dev] = true;
        }
        if(nimages == 0)
            return cudaSuccess;
        if(nimages > 0x7fffffffull)
            return cudaErrorInvalidConfiguration;
        kern<<<(unsigned)nimages, F::THREADS, F::SMEM_BYTES, stream>>>(a);
        return cudaGetLastError();
    }
} // namespace b200fft
