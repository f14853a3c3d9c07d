// Bluestein's algorithm for one long prime-ish row per CTA, with the padded length M = R x 1024
// laid out as R rows of 1024 points and ONE WARP PER ROW.
//
// Role in the reference: library/src/tree_node_bluestein.cpp (chirp multiply, FFT_M, filter
// multiply, IFFT_M, chirp multiply; docs/design/bluestein.rst:20-31, 159-191), which runs the
// M-point transforms as separate kernels through a work buffer for lengths of this size.
//
// Why this shape.  The three-pass form of the M-point transform (stockham_engine.cuh,
// bluestein_tile_kernel) makes all 20 warps of the single resident CTA walk through six passes
// in lockstep, two CTA-wide barriers each, and spends two thirds of its time waiting.  Here the
// M-point transform is the classic two-level split n = n1 + 1024 n2, k = R k1 + k2:
//
//   columns   thread per n1: the R-point DFT over n2.  Bluestein's input is zero from M/2 on, so only
//             n2 < R/2 is non-zero and the R-point DFT is two R/2-point butterflies (even k2 from the
//             inputs, odd k2 from the inputs times W_R^n2); times W_M^(n1 k2); into the shared tile [k2][n1];
//   rows      warp k2: the 1024-point transform over n1 as 32 x 32 with one point column per lane and the
//             exchange inside the warp (no CTA barrier), times the filter (stored [k2][k1] by the host),
//             the inverse 1024-point transform the same way, back into the tile;
//   columns   thread per m1: times conj W_M^(m1 k2), then the inverse R-point DFT over k2, of which only the outputs m2 < R/2 are
//             wanted (again two R/2-point butterflies), times the chirp, to global memory.
//
// Two CTA barriers per transform instead of twelve; in the row phase, which is most of the work,
// every warp runs on its own.  Inverse transforms exchange real and imaginary parts on load and on
// store (gload / gstore), as everywhere in this library.
//
// kargs: as bluestein_tile_kernel — iaux[0] = n, aux[0] = chirp (n entries), aux[1] = filter in
// [k2][k1] order (M entries, 1/M folded in), aux[2] = W_M^(n1 k2) in [k2][n1] order (M entries),
// twiddles = stacked table of the 1024-point transform (32 x 32: 992 entries).
#pragma once
#include "stockham_engine.cuh"

namespace b200fft
{
    template <int R, typename T = float>
    struct BlueRC
    {
        static constexpr int    CN         = 1024; // points per row
        static constexpr int    M          = R * CN;
        static constexpr int    H          = R / 2;
        static constexpr int    THREADS    = 32 * R;
        static constexpr size_t TILE_BYTES = (size_t)M * 2 * sizeof(T);
        static constexpr int    TW_ENTRIES = 31 * 32;
        static constexpr size_t SMEM_BYTES = TILE_BYTES + (size_t)TW_ENTRIES * 2 * sizeof(T);
        // resident CTAs per SM the launch bounds ask for: what shared memory allows, as long as ~85 registers remain
        static constexpr int MINB = sizeof(T) == 8 ? 1 : (R <= 6 ? 3 : (R <= 12 ? 2 : 1)); // (32 double-precision points per lane: ~200 registers)
        static_assert(R % 2 == 0 && R >= 4 && R <= 32, "even row counts up to 32");
    };

    // forward 1024-point transform held by one warp: lane t has points t + 32 j in r[j] on entry and on exit.
    // `xw` = 1056 components of shared memory private to the warp; `tws` = W_1024^(j t) at [(j-1) * 32 + t].
    template <typename T, typename T2>
    __device__ __forceinline__ void warp_fft1024(T2 (&r)[32], T* xw, const T2* tws, const int lane)
    {
        Butterfly<32, T2>::run(r);
#pragma unroll
        for(int half = 0; half < 2; ++half)
        {
            __syncwarp();
#pragma unroll
            for(int j = 0; j < 32; ++j)
            {
                const int e            = 32 * lane + j;
                xw[e + (e >> 5)]       = half == 0 ? r[j].x : r[j].y;
            }
            __syncwarp();
#pragma unroll
            for(int j = 0; j < 32; ++j)
            {
                const int   e = lane + 32 * j;
                const T     v = xw[e + (e >> 5)];
                if(half == 0)
                    r[j].x = v;
                else
                    r[j].y = v;
            }
        }
#pragma unroll
        for(int j = 1; j < 32; ++j)
            r[j] = cmul(r[j], tws[(j - 1) * 32 + lane]);
        Butterfly<32, T2>::run(r);
    }

    template <class C, int R>
    __global__ void __launch_bounds__(32 * R, (BlueRC<R, typename C::T>::MINB)) bluestein_rc_kernel(const __grid_constant__ b200fft_kargs a)
    {
        using T  = typename C::T;
        using B  = BlueRC<R, T>;
        using T2 = typename C::T2;
        constexpr int CN = B::CN, H = B::H;
        extern __shared__ __align__(16) unsigned char smem_raw[];
        T2* tile = reinterpret_cast<T2*>(smem_raw);
        T2* tws  = reinterpret_cast<T2*>(smem_raw + B::TILE_BYTES);

        const int     tid     = threadIdx.x;
        const int     lane    = tid & 31;
        const int     warp    = tid >> 5;
        const TilePos tp      = decode_tile(a, blockIdx.x, 1);
        const bool    inverse = a.inverse != 0;
        const bool    use_sc  = a.use_scale != 0;
        const T       scale   = (T)a.scale;
        const int     n       = (int)a.iaux[0];
        const T2* __restrict__ tw    = reinterpret_cast<const T2*>(a.twiddles);
        const T2* __restrict__ chirp = reinterpret_cast<const T2*>(a.aux[0]);
        const T2* __restrict__ filt  = reinterpret_cast<const T2*>(a.aux[1]);
        const T2* __restrict__ twm   = reinterpret_cast<const T2*>(a.aux[2]);
        const long long ibase = view_base(a.in, tp.i0_first, tp.i1, tp.i2);
        const long long obase = view_base(a.out, tp.i0_first, tp.i1, tp.i2);

        for(int i = tid; i < B::TW_ENTRIES; i += B::THREADS)
            tws[i] = tw[i];
        // W_R^j, j < R/2
        T2 wr[H];
#pragma unroll
        for(int j = 0; j < H; ++j)
        {
            double s, c;
            sincospi(2.0 * (double)j / (double)R, &s, &c);
            wr[j].x = (T)c;
            wr[j].y = (T)(-s);
        }

        // ---- columns, forward (the loads of all of a thread's columns are issued before any arithmetic) ----
        constexpr int ROUNDS = (CN + B::THREADS - 1) / B::THREADS;
        {
            // Every load of the input is issued before anything depends on one: clamped indices instead of
            // branches (points past the end are read from the last point and zeroed afterwards), the planar /
            // interleaved decision outside the loops.  With a branch and a multiply behind each load the
            // twenty device-memory round trips of a thread ran one after the other (measured: 19 000 of the
            // phase's 25 000 cycles).
            T2 v[ROUNDS][H];
            const long long es = a.in.es;
            if(a.in.planar)
            {
                const T* __restrict__ p0 = reinterpret_cast<const T*>(a.in.p[0]);
                const T* __restrict__ p1 = reinterpret_cast<const T*>(a.in.p[1]);
#pragma unroll
                for(int q = 0; q < ROUNDS; ++q)
#pragma unroll
                    for(int j = 0; j < H; ++j)
                    {
                        const int       e   = min(min(tid + q * B::THREADS, CN - 1) + CN * j, n - 1);
                        const long long off = ibase + (long long)e * es;
                        v[q][j].x           = p0[off];
                        v[q][j].y           = p1[off];
                    }
            }
            else
            {
                const T2* __restrict__ p0 = reinterpret_cast<const T2*>(a.in.p[0]);
#pragma unroll
                for(int q = 0; q < ROUNDS; ++q)
#pragma unroll
                    for(int j = 0; j < H; ++j)
                    {
                        const int e = min(min(tid + q * B::THREADS, CN - 1) + CN * j, n - 1);
                        v[q][j]     = p0[ibase + (long long)e * es];
                    }
            }
#pragma unroll
            for(int q = 0; q < ROUNDS; ++q)
            {
                T2 ch[H];
#pragma unroll
                for(int j = 0; j < H; ++j)
                    ch[j] = chirp[min(min(tid + q * B::THREADS, CN - 1) + CN * j, n - 1)];
#pragma unroll
                for(int j = 0; j < H; ++j)
                {
                    const bool live = tid + q * B::THREADS + CN * j < n;
                    const T2   x    = inverse ? cswap(v[q][j]) : v[q][j];
                    const T2   y    = cmul(x, ch[j]);
                    v[q][j].x       = live ? y.x : (T)0;
                    v[q][j].y       = live ? y.y : (T)0;
                }
            }
#pragma unroll
            for(int q = 0; q < ROUNDS; ++q)
            {
                const int c = tid + q * B::THREADS;
                if(c < CN)
                {
                    T2 w[H];
#pragma unroll
                    for(int j = 0; j < H; ++j)
                        w[j] = cmul(v[q][j], wr[j]);
                    Butterfly<H, T2>::run(v[q]);
                    Butterfly<H, T2>::run(w);
#pragma unroll
                    for(int m = 0; m < H; ++m)
                    {
                        tile[(2 * m) * CN + c]     = cmul(v[q][m], twm[(2 * m) * CN + c]);
                        tile[(2 * m + 1) * CN + c] = cmul(w[m], twm[(2 * m + 1) * CN + c]);
                    }
                }
            }
        }
        __syncthreads();

        // ---- rows: forward transform, filter, inverse transform; one warp per row ----
        {
            T2*    row = tile + warp * CN;
            T*     xw  = reinterpret_cast<T*>(row);
            T2     r[32];
#pragma unroll
            for(int j = 0; j < 32; ++j)
                r[j] = row[lane + 32 * j];
            const T2* __restrict__ f = filt + warp * CN;
            if constexpr(R >= 20)
            {
                // one copy of the transform's code for both directions: at 640 threads (96 registers) four
                // radix-32 butterflies per thread in a straight line overflowed the instruction cache — 10007
                // points, 4096 transforms: 0.667 -> 0.573 ms.  (With fewer rows the straight-line form below is
                // faster, 16 rows by 11 %; rolling the column loops the same way cost more in spills and
                // serialised loads than it saved.)
#pragma unroll 1
                for(int dir = 0; dir < 2; ++dir)
                {
                    warp_fft1024(r, xw, tws, lane);
                    if(dir == 0)
                    {
#pragma unroll
                        for(int j = 0; j < 32; ++j)
                            r[j] = cswap(cmul(r[j], f[lane + 32 * j]));
                    }
                }
            }
            else
            {
                warp_fft1024(r, xw, tws, lane);
#pragma unroll
                for(int j = 0; j < 32; ++j)
                    r[j] = cswap(cmul(r[j], f[lane + 32 * j]));
                warp_fft1024(r, xw, tws, lane);
            }
            __syncwarp();
#pragma unroll
            for(int j = 0; j < 32; ++j)
                row[lane + 32 * j] = r[j]; // parts still exchanged and the twiddle still owed: the column phase does both
        }
        // the twiddles and chirp values of this thread's first column travel while the barrier is waited for
        T2 tv[R], cv[H];
#pragma unroll
        for(int k = 0; k < R; ++k)
            tv[k] = twm[k * CN + tid];
#pragma unroll
        for(int m2 = 0; m2 < H; ++m2)
            cv[m2] = (tid + CN * m2 < n) ? chirp[tid + CN * m2] : T2{(T)0, (T)0};
        __syncthreads();

        // ---- columns, inverse; outputs m2 < R/2 only ----
#pragma unroll
        for(int q = 0; q < ROUNDS; ++q)
        {
            const int c = tid + q * B::THREADS;
            if(c < CN)
            {
                if(q > 0)
                {
#pragma unroll
                    for(int k = 0; k < R; ++k)
                        tv[k] = twm[k * CN + c];
#pragma unroll
                    for(int m2 = 0; m2 < H; ++m2)
                        cv[m2] = (c + CN * m2 < n) ? chirp[c + CN * m2] : T2{(T)0, (T)0};
                }
                T2 ev[H], od[H];
#pragma unroll
                for(int m = 0; m < H; ++m)
                {
                    // tile holds swap(U); V = U conj(W_M^(m1 k2)); the R/2-point inverse DFTs run on swap(V)
                    ev[m] = cswap(cmulc(cswap(tile[(2 * m) * CN + c]), tv[2 * m]));
                    od[m] = cswap(cmulc(cswap(tile[(2 * m + 1) * CN + c]), tv[2 * m + 1]));
                }
                Butterfly<H, T2>::run(ev);
                Butterfly<H, T2>::run(od);
#pragma unroll
                for(int m2 = 0; m2 < H; ++m2)
                {
                    const int e = c + CN * m2;
                    if(e < n)
                    {
                        const T2 o = cmulc(cswap(od[m2]), wr[m2]);
                        T2       y = cswap(ev[m2]);
                        y.x += o.x;
                        y.y += o.y;
                        gstore<C>(a.out, obase, e, cmul(y, cv[m2]), inverse, use_sc, scale);
                    }
                }
            }
        }
    }

    template <class C, int R>
    cudaError_t launch_bluestein_rc_kernel(const b200fft_kargs& a, unsigned long long ntiles, cudaStream_t stream)
    {
        using B = BlueRC<R, typename C::T>;
        static std::atomic<bool> attr_done[64]; // zero-initialised; host threads may launch the same kernel concurrently
        int                      dev = 0;
        cudaGetDevice(&dev);
        if(dev < 64 && !attr_done[dev])
        {
            cudaError_t e = cudaFuncSetAttribute(bluestein_rc_kernel<C, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)B::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            attr_done[dev] = true;
        }
        if(ntiles == 0)
            return cudaSuccess;
        if(ntiles > 0x7fffffffull || !a.aux[0] || !a.aux[1] || !a.aux[2])
            return cudaErrorInvalidConfiguration;
        bluestein_rc_kernel<C, R><<<(unsigned)ntiles, B::THREADS, B::SMEM_BYTES, stream>>>(a);
        return cudaGetLastError();
    }
} // namespace b200fft
