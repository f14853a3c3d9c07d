// Stockham autosort FFT engine for sm_100a: one CTA transforms a tile of TPB
// batched 1D transforms of compile-time length N held in shared memory.
//
// Role in the reference: library/src/device/generator/stockham_gen_base.h:642-918
// (the generated kernel body), stockham_gen_rr.h / _cc.h / _rc.h / _cr.h (the
// four tiling modes: row/column input x row/column output) and the
// load/twiddle/butterfly/store generators at :347-456.  This file is the
// hand-written device-side half; the offline generator instantiates it with
// explicit factor lists and supplies the straight-line butterflies.
//
// Pass structure (same decomposition the reference uses, restated):
//   pass p has radix W = F[p], height CH = F[0]*...*F[p-1], NB = N/W butterflies.
//   butterfly b reads points b + j*NB (j < W), multiplies point j >= 1 by
//   exp(-2 pi i * j * (b mod CH) / (CH*W)), runs the radix-W DFT and writes
//   result j to (b div CH)*W*CH + (b mod CH) + j*CH.  After the last pass the
//   data is in natural order.
//
// Thread mapping:
//   ROW tiles:  thread = c*TPT + t   (c = transform in tile, t = lane in transform),
//               shared layout [c][pad(e)], coalesced along the transform.
//   COL tiles:  thread = t*TPB + c,  shared layout [e][c], coalesced across the
//               TPB adjacent transforms (column FFTs of 2D/3D data).
//   Pass 0 reads global memory straight into registers and the last pass
//   writes registers straight to global memory, so a kernel makes one HBM
//   round trip; optional cooperative stages re-map threads for transposing
//   loads/stores.
#pragma once
#include "fft_types.cuh"
#include "kargs.h"
#include <atomic>
#include <cuda_runtime.h>

namespace b200fft
{
    // compile-time factor list
    template <int... F>
    struct FactorList
    {
        static constexpr int count = sizeof...(F);
        __host__ __device__ static constexpr int get(int i)
        {
            constexpr int v[] = {F...};
            return v[i];
        }
        __host__ __device__ static constexpr int cum(int i)
        {
            int c = 1;
            for(int k = 0; k < i; ++k)
                c *= get(k);
            return c;
        }
        // offset of pass p's block inside the stacked twiddle table
        // (pass 0 has no twiddles; pass p holds (W-1)*CH entries)
        __host__ __device__ static constexpr int tw_offset(int p)
        {
            int o = 0;
            for(int k = 1; k < p; ++k)
                o += (get(k) - 1) * cum(k);
            return o;
        }
    };

    enum IoKind
    {
        IO_UNIT    = 0, // interleaved complex, unit stride along the transform (both sides)
        IO_STRIDED = 1, // interleaved complex, run-time strides
        IO_GENERIC = 2, // interleaved or planar chosen at run time, run-time strides
        IO_BLKOUT  = 3, // like IO_STRIDED, output with a two-level stride along the transform
        // real transforms computed as full-length complex ones (odd lengths; reference: the odd-length
        // real kernels of library/src/device/generator and rtc_realcomplex_gen.cpp "r2c_copy"/"c2r_copy" paths)
        IO_REAL_IN  = 4, // input: real scalars, run-time stride; imaginary part taken as zero
        IO_HERM_OUT = 5, // output: generic complex store of the points 0..N/2 only
        IO_HERM_IN  = 6, // input: points 0..N/2 given; point e > N/2 is the conjugate of point N-e
        IO_REAL_OUT = 7, // output: real part only, run-time stride
    };
    enum CoopKind
    {
        COOP_NONE  = 0, // pass threads touch global memory themselves
        COOP_EFAST = 1, // staged through shared memory, consecutive threads walk a transform
        COOP_CFAST = 2, // staged, consecutive threads walk across the tile's transforms
        // even-length real transforms fused into the half-length complex kernel
        // (reference: library/src/rtc_realcomplex_gen.cpp:348-573, fused there only below length 512)
        COOP_R2C_POST = 3, // output stage: Hermitian post-processing of the packed FFT
        COOP_C2R_PRE  = 4, // input stage: Hermitian pre-processing into the packed FFT
    };

    // Kernel configuration; instantiated by generated code.
    template <typename T_,
              int  N_,
              int  TPT_,
              int  TPB_,
              bool COL_,
              int  IOKI_,
              int  IOKO_,
              int  CIN_,
              int  COUT_,
              int  MINB_,
              class FL_>
    struct KCfg
    {
        using T  = T_;
        using T2 = typename cx<T_>::type;
        using TW2 = typename twof<T_>::type; // entries of the twiddle tables
        using FL = FL_;
        static constexpr int  N       = N_;
        static constexpr int  TPT     = TPT_;
        static constexpr int  TPB     = TPB_;
        static constexpr bool COL     = COL_;
        static constexpr int  IOKI    = IOKI_; // addressing of the input side
        static constexpr int  IOKO    = IOKO_; // addressing of the output side
        static constexpr int  CIN     = CIN_;
        static constexpr int  COUT    = COUT_;
        static constexpr int  MINB    = MINB_;
        static constexpr int  THREADS = TPT_ * TPB_;
        static constexpr int  NPASS   = FL_::count;
        // row layout: one pad element every 128 bytes, and an odd row pitch so
        // that walking across rows is conflict-free as well
        static constexpr int PADSHIFT = (sizeof(T_) == 4) ? 4 : 3;
        static constexpr int NPAD     = COL_ ? N_ : ((N_ + (N_ >> PADSHIFT)) | 1);
        static constexpr int SMEM_ELEMS = COL_ ? N_ * TPB_ : NPAD * TPB_;
        static constexpr bool NEEDS_SMEM = (NPASS > 1) || CIN_ != COOP_NONE || COUT_ != COOP_NONE;
        static constexpr size_t SMEM_BYTES
            = NEEDS_SMEM ? sizeof(T2) * (size_t)SMEM_ELEMS + (CIN_ != COOP_NONE || COUT_ != COOP_NONE ? 16 * TPB_ : 0)
                         : 0;

        __device__ static __forceinline__ int sidx(int c, int e)
        {
            if constexpr(COL_)
                return e * TPB_ + c;
            else
                return c * NPAD + e + (e >> PADSHIFT);
        }
    };

    // ------------------------------------------------------------------
    // global-memory element access
    // ------------------------------------------------------------------
    // offset of point e of a transform along a two-level stride (v.blk >= 2)
    __device__ __forceinline__ long long elem_offset(const b200fft_ioview& v, int e)
    {
        const unsigned q = __umulhi((unsigned)e, v.blk_mul);
        const unsigned r = (unsigned)e - q * v.blk;
        return (long long)q * v.bs + (long long)r * v.es;
    }

    // address of point e of a blocked output: either inside the local buffer or, with a
    // per-block pointer table, inside the buffer of the rank that owns the block
    template <typename T2>
    __device__ __forceinline__ T2* blk_address(const b200fft_ioview& v, long long base, int e)
    {
        const unsigned q = __umulhi((unsigned)e, v.blk_mul);
        const unsigned r = (unsigned)e - q * v.blk;
        if(v.blk_ptrs)
            return reinterpret_cast<T2*>(v.blk_ptrs[q]) + base + (long long)r * v.es;
        return reinterpret_cast<T2*>(v.p[0]) + base + (long long)q * v.bs + (long long)r * v.es;
    }

    template <class C>
    __device__ __forceinline__ typename C::T2
        gload(const b200fft_ioview& v, long long base, int e, bool inverse)
    {
        using T  = typename C::T;
        using T2 = typename C::T2;
        T2 r;
        if constexpr(C::IOKI == IO_UNIT)
        {
            r = reinterpret_cast<const T2*>(v.p[0])[base + e];
        }
        else if constexpr(C::IOKI == IO_STRIDED || C::IOKI == IO_BLKOUT)
        {
            r = reinterpret_cast<const T2*>(v.p[0])[base + (long long)e * v.es];
        }
        else if constexpr(C::IOKI == IO_REAL_IN)
        {
            r.x = reinterpret_cast<const T*>(v.p[0])[base + (long long)e * v.es];
            r.y = 0;
        }
        else if constexpr(C::IOKI == IO_HERM_IN)
        {
            const bool      upper = e > C::N / 2;
            const int       ee    = upper ? C::N - e : e;
            const long long off   = base + (long long)ee * v.es;
            if(v.planar)
            {
                r.x = reinterpret_cast<const T*>(v.p[0])[off];
                r.y = reinterpret_cast<const T*>(v.p[1])[off];
            }
            else
                r = reinterpret_cast<const T2*>(v.p[0])[off];
            if(upper)
                r.y = -r.y;
            // the imaginary parts of DC and Nyquist carry no information
            if(ee == 0 || (C::N % 2 == 0 && ee == C::N / 2))
                r.y = 0;
        }
        else
        {
            const long long off = base + (long long)e * v.es;
            if(v.planar)
            {
                r.x = reinterpret_cast<const T*>(v.p[0])[off];
                r.y = reinterpret_cast<const T*>(v.p[1])[off];
            }
            else
                r = reinterpret_cast<const T2*>(v.p[0])[off];
        }
        return inverse ? cswap(r) : r;
    }

    template <class C>
    __device__ __forceinline__ void gstore(const b200fft_ioview& v,
                                           long long             base,
                                           int                   e,
                                           typename C::T2        val,
                                           bool                  inverse,
                                           bool                  use_scale,
                                           typename C::T         scale)
    {
        using T  = typename C::T;
        using T2 = typename C::T2;
        if(inverse)
            val = cswap(val);
        if(use_scale)
        {
            val.x *= scale;
            val.y *= scale;
        }
        if constexpr(C::IOKO == IO_UNIT)
        {
            reinterpret_cast<T2*>(v.p[0])[base + e] = val;
        }
        else if constexpr(C::IOKO == IO_STRIDED)
        {
            reinterpret_cast<T2*>(v.p[0])[base + (long long)e * v.es] = val;
        }
        else if constexpr(C::IOKO == IO_BLKOUT)
        {
            *blk_address<T2>(v, base, e) = val;
        }
        else if constexpr(C::IOKO == IO_REAL_OUT)
        {
            reinterpret_cast<T*>(v.p[0])[base + (long long)e * v.es] = val.x;
        }
        else if constexpr(C::IOKO == IO_HERM_OUT)
        {
            if(e <= C::N / 2)
            {
                const long long off = base + (long long)e * v.es;
                if(v.planar)
                {
                    reinterpret_cast<T*>(v.p[0])[off] = val.x;
                    reinterpret_cast<T*>(v.p[1])[off] = val.y;
                }
                else
                    reinterpret_cast<T2*>(v.p[0])[off] = val;
            }
        }
        else
        {
            const long long off = base + (long long)e * v.es;
            if(v.planar)
            {
                reinterpret_cast<T*>(v.p[0])[off] = val.x;
                reinterpret_cast<T*>(v.p[1])[off] = val.y;
            }
            else
                reinterpret_cast<T2*>(v.p[0])[off] = val;
        }
    }

    // W_N^u from a stepped table: `steps` sub-tables of 256 entries, sub-table s
    // holding exp(-2 pi i * j * 256^s / N)
    template <typename T2>
    __device__ __forceinline__ T2 large_twiddle(const T2* __restrict__ tab, unsigned long long u, int steps)
    {
        T2 w = tab[u & 255];
        for(int s = 1; s < steps; ++s)
        {
            u >>= 8;
            w = cmul(w, tab[256 * s + (u & 255)]);
        }
        return w;
    }


#ifndef B200FFT_TW4_MIN
#define B200FFT_TW4_MIN 2048 // shortest transform whose passes factor their twiddle loads
#endif

    // ------------------------------------------------------------------
    // one radix pass
    // ------------------------------------------------------------------
    template <class C, int P, class LD, class ST>
    __device__ __forceinline__ void
        run_pass(const int t, LD ld, ST st, const typename C::TW2* __restrict__ tw, const bool sync_mid)
    {
        using T2          = typename C::T2;
        using TW2         = typename C::TW2;
        constexpr int W   = C::FL::get(P);
        constexpr int CH  = C::FL::cum(P);
        constexpr int NB  = C::N / W;
        constexpr int BPT = (NB + C::TPT - 1) / C::TPT;
        constexpr bool FULL = (NB % C::TPT) == 0;
        constexpr int TWO = C::FL::tw_offset(P);

        // Long transforms: the stacked table no longer fits the L1 left beside the shared tile, so
        // twiddle loads come from L2.  Load only the legs j = 1,2,3 and j = 4a and form the others as
        // products (j = 4a + b): 6 instead of 15 loads for radix 16, 10 instead of 31 for radix 32, at
        // the cost of one complex multiply per remaining leg (error of one extra rounding, far inside
        // the bound) — and issue those loads BEFORE the data loads and the barrier, so that their L2
        // latency overlaps both instead of following the barrier.
        constexpr bool TW4 = (P > 0) && (C::N >= B200FFT_TW4_MIN) && (W >= 8);
        constexpr int  NA  = TW4 ? (W - 1) / 4 : 1; // legs 4, 8, ...
        TW2 wb[BPT][3], wa[BPT][NA];
        if constexpr(TW4)
        {
#pragma unroll
            for(int i = 0; i < BPT; ++i)
            {
                const int b = t + i * C::TPT;
                if(FULL || b < NB)
                {
                    const int k = b % CH;
#pragma unroll
                    for(int b4 = 1; b4 < 4; ++b4)
                        wb[i][b4 - 1] = tw[TWO + (b4 - 1) * CH + k];
#pragma unroll
                    for(int a4 = 1; 4 * a4 < W; ++a4)
                        wa[i][a4 - 1] = tw[TWO + (4 * a4 - 1) * CH + k];
                }
            }
        }
        T2 x[BPT][W];
#pragma unroll
        for(int i = 0; i < BPT; ++i)
        {
            const int b = t + i * C::TPT;
            if(FULL || b < NB)
            {
#pragma unroll
                for(int j = 0; j < W; ++j)
                    x[i][j] = ld(b + j * NB);
            }
        }
        if(sync_mid)
            __syncthreads();
#pragma unroll
        for(int i = 0; i < BPT; ++i)
        {
            const int b = t + i * C::TPT;
            if(FULL || b < NB)
            {
                const int k = b % CH;
                if constexpr(P > 0)
                {
                    if constexpr(TW4)
                    {
#pragma unroll
                        for(int b4 = 1; b4 < 4; ++b4)
                            x[i][b4] = tmul(x[i][b4], wb[i][b4 - 1]);
#pragma unroll
                        for(int a4 = 1; 4 * a4 < W; ++a4)
                        {
                            x[i][4 * a4] = tmul(x[i][4 * a4], wa[i][a4 - 1]);
#pragma unroll
                            for(int b4 = 1; b4 < 4; ++b4)
                                if(4 * a4 + b4 < W)
                                    x[i][4 * a4 + b4] = tmul(x[i][4 * a4 + b4], cmul(wa[i][a4 - 1], wb[i][b4 - 1]));
                        }
                    }
                    else
                    {
#pragma unroll
                        for(int j = 1; j < W; ++j)
                            x[i][j] = tmul(x[i][j], tw[TWO + (j - 1) * CH + k]);
                    }
                }
                Butterfly<W, T2>::run(x[i]);
                const int base = (b / CH) * (W * CH) + k;
#pragma unroll
                for(int j = 0; j < W; ++j)
                    st(base + j * CH, x[i][j]);
            }
        }
    }

    // Runs passes FIRST..NPASS-1 recursively.  `src`/`dst` are the first
    // pass's loader and the last pass's storer; middle traffic goes through
    // shared memory.  SRC_SMEM / DST_SMEM tell whether src / dst alias the
    // shared tile (then barriers are needed around them).
    template <class C, int P, bool SRC_SMEM, bool DST_SMEM, class SRC, class DST>
    __device__ __forceinline__ void run_passes(const int                 t,
                                               const int                 c,
                                               typename C::T2*           sm,
                                               const typename C::TW2* __restrict__ tw,
                                               SRC                       src,
                                               DST                       dst)
    {
        using T2                 = typename C::T2;
        constexpr bool first     = (P == 0);
        constexpr bool last      = (P == C::NPASS - 1);
        auto           sm_load   = [=](int e) -> T2 { return sm[C::sidx(c, e)]; };
        auto           sm_store  = [=](int e, T2 v) { sm[C::sidx(c, e)] = v; };
        constexpr bool rd_smem   = first ? SRC_SMEM : true;
        constexpr bool wr_smem   = last ? DST_SMEM : true;
        constexpr bool sync_mid  = rd_smem && wr_smem;

        if constexpr(first && last)
            run_pass<C, P>(t, src, dst, tw, sync_mid);
        else if constexpr(first)
            run_pass<C, P>(t, src, sm_store, tw, sync_mid);
        else if constexpr(last)
            run_pass<C, P>(t, sm_load, dst, tw, sync_mid);
        else
            run_pass<C, P>(t, sm_load, sm_store, tw, sync_mid);

        if constexpr(wr_smem)
            __syncthreads();
        if constexpr(!last)
            run_passes<C, P + 1, SRC_SMEM, DST_SMEM>(t, c, sm, tw, src, dst);
    }

    // ------------------------------------------------------------------
    // tile bookkeeping
    // ------------------------------------------------------------------
    struct TilePos
    {
        unsigned i0_first; // first outer-0 index of the tile
        unsigned i1, i2;
    };

    __device__ __forceinline__ TilePos decode_tile(const b200fft_kargs& a, unsigned tile, int tpb)
    {
        TilePos  p;
        unsigned t0 = tile % a.ntile0;
        unsigned r  = tile / a.ntile0;
        p.i0_first  = t0 * (unsigned)tpb;
        p.i1        = r % a.on[1];
        p.i2        = r / a.on[1];
        return p;
    }

    __device__ __forceinline__ long long
        view_base(const b200fft_ioview& v, unsigned i0, unsigned i1, unsigned i2)
    {
        return (long long)i0 * v.os[0] + (long long)i1 * v.os[1] + (long long)i2 * v.os[2];
    }

    // ------------------------------------------------------------------
    // the kernel
    // ------------------------------------------------------------------
    template <class C>
    __global__ void __launch_bounds__(C::THREADS, C::MINB)
        stockham_tile_kernel(const __grid_constant__ b200fft_kargs a)
    {
        using T  = typename C::T;
        using T2 = typename C::T2;
        extern __shared__ __align__(16) unsigned char smem_raw[];
        T2* sm = reinterpret_cast<T2*>(smem_raw);

        const int tid = threadIdx.x;
        int       c, t;
        if constexpr(C::COL)
        {
            c = tid % C::TPB;
            t = tid / C::TPB;
        }
        else
        {
            c = tid / C::TPT;
            t = tid % C::TPT;
        }
        const TilePos  tp      = decode_tile(a, blockIdx.x, C::TPB);
        const bool     inverse = a.inverse != 0;
        const bool     use_sc  = a.use_scale != 0;
        const T        scale   = (T)a.scale;
        const T2* __restrict__ tw = reinterpret_cast<const T2*>(a.twiddles);

        // per-transform base offsets for cooperative stages
        long long* bases = reinterpret_cast<long long*>(smem_raw + sizeof(T2) * (size_t)C::SMEM_ELEMS);
        if constexpr(C::CIN != COOP_NONE || C::COUT != COOP_NONE)
        {
            if(tid < C::TPB)
            {
                bases[2 * tid]     = view_base(a.in, tp.i0_first + tid, tp.i1, tp.i2);
                bases[2 * tid + 1] = view_base(a.out, tp.i0_first + tid, tp.i1, tp.i2);
            }
            __syncthreads();
        }
        const unsigned nvalid = min((unsigned)C::TPB, a.on[0] - tp.i0_first);

        const bool      valid = (unsigned)c < nvalid;
        const long long ibase = view_base(a.in, tp.i0_first + c, tp.i1, tp.i2);
        const long long obase = view_base(a.out, tp.i0_first + c, tp.i1, tp.i2);

        // ---- cooperative load stage ----
        if constexpr(C::CIN == COOP_C2R_PRE)
        {
            // in: Hermitian rows X[0..h] (h = N); shared memory receives Z' with
            // Z'_p = (X_p + conj X_q) + i conj(W^p) (X_p - conj X_q),  q = h - p,
            // whose unnormalised inverse FFT is the packed real row.  Stored with
            // parts exchanged: the forward passes then compute the inverse.
            constexpr int H     = C::N;
            constexpr int NP    = H / 2 + 1;
            constexpr int ITEMS = NP * C::TPB;
            constexpr int ITER  = (ITEMS + C::THREADS - 1) / C::THREADS;
            constexpr int UNR   = ITER < 8 ? ITER : 8; // loads in flight per thread
            const T2* __restrict__ htw = reinterpret_cast<const T2*>(a.aux[0]);
            for(int it0 = 0; it0 < ITER; it0 += UNR)
            {
                T2 xa[UNR], xb[UNR], w[UNR];
#pragma unroll
                for(int u = 0; u < UNR; ++u)
                {
                    const int idx = tid + (it0 + u) * C::THREADS;
                    const int cc  = idx / NP;
                    const int p   = idx % NP;
                    xa[u].x = xa[u].y = xb[u].x = xb[u].y = 0;
                    w[u].x = w[u].y = 0;
                    if(idx < ITEMS && (unsigned)cc < nvalid)
                    {
                        xa[u] = gload<C>(a.in, bases[2 * cc], p, false);
                        xb[u] = gload<C>(a.in, bases[2 * cc], H - p, false);
                        w[u]  = htw[p];
                    }
                }
#pragma unroll
                for(int u = 0; u < UNR; ++u)
                {
                    const int idx = tid + (it0 + u) * C::THREADS;
                    if(idx >= ITEMS)
                        continue;
                    const int cc = idx / NP;
                    const int p  = idx % NP;
                    const int q  = H - p;
                    T2        a0 = xa[u], b0 = xb[u];
                    if(p == 0)
                    {
                        a0.y = 0; // imaginary parts of DC and Nyquist carry no information
                        b0.y = 0;
                    }
                    b0.y = -b0.y;
                    T2 e, d, t;
                    e.x = a0.x + b0.x;
                    e.y = a0.y + b0.y;
                    d.x = a0.x - b0.x;
                    d.y = a0.y - b0.y;
                    t.x = w[u].y; // i * conj(W^p)
                    t.y = w[u].x;
                    const T2 td = cmul(t, d);
                    T2       zp, zq;
                    zp.x = e.x + td.x;
                    zp.y = e.y + td.y;
                    zq.x = e.x - td.x;
                    zq.y = -(e.y - td.y);
                    sm[C::sidx(cc, p)] = cswap(zp);
                    if(p != q && p != 0)
                        sm[C::sidx(cc, q)] = cswap(zq);
                }
            }
            __syncthreads();
        }
        else if constexpr(C::CIN != COOP_NONE)
        {
            constexpr int ITEMS = C::N * C::TPB;
            constexpr int ITER  = (ITEMS + C::THREADS - 1) / C::THREADS;
            constexpr int UNR   = ITER < 8 ? ITER : 8; // loads in flight per thread
            for(int it0 = 0; it0 < ITER; it0 += UNR)
            {
                T2 v[UNR];
#pragma unroll
                for(int u = 0; u < UNR; ++u)
                {
                    const int idx = tid + (it0 + u) * C::THREADS;
                    const int cc  = (C::CIN == COOP_EFAST) ? idx / C::N : idx % C::TPB;
                    const int e   = (C::CIN == COOP_EFAST) ? idx % C::N : idx / C::TPB;
                    v[u].x = v[u].y = 0;
                    if(idx < ITEMS && (unsigned)cc < nvalid)
                        v[u] = gload<C>(a.in, bases[2 * cc], e, inverse);
                }
#pragma unroll
                for(int u = 0; u < UNR; ++u)
                {
                    const int idx = tid + (it0 + u) * C::THREADS;
                    const int cc  = (C::CIN == COOP_EFAST) ? idx / C::N : idx % C::TPB;
                    const int e   = (C::CIN == COOP_EFAST) ? idx % C::N : idx / C::TPB;
                    if(idx < ITEMS)
                        sm[C::sidx(cc, e)] = v[u];
                }
            }
            __syncthreads();
        }

        // Second kernel of a long 1D transform (n = n1 * n2, this kernel: length n2 for each k1): the
        // N1 x N2 twiddle multiply W_n^(k1 * e) rides on the loads of the variants used there
        // (reference: large twiddles fused into the SBCC kernels, library/src/device/kernels/common.h:227-301).
        // aux[2] = stepped table of three 256-entry sub-tables; k1 = this transform's index along outer dimension 0.
        // The value was loaded with parts exchanged for an inverse transform, for which the product
        // with the forward factor is exactly the exchanged product with the conjugate factor.
        constexpr bool LT_CAPABLE = !C::COL && C::CIN == COOP_NONE && (C::IOKI == IO_GENERIC || C::COUT == COOP_CFAST);
        const T2* __restrict__ lt_tab = LT_CAPABLE ? reinterpret_cast<const T2*>(a.aux[2]) : nullptr;
        const unsigned long long lt_k1 = tp.i0_first + (unsigned)c;
        auto g_src = [&](int e) -> T2 {
            T2 v;
            v.x = 0;
            v.y = 0;
            if(valid)
                v = gload<C>(a.in, ibase, e, inverse);
            return v;
        };
        // branch-free: the table always has three sub-tables (unused ones hold 1), so that the loads of a
        // pass still issue back to back
        auto g_src_lt = [&](int e) -> T2 {
            T2 v;
            v.x = 0;
            v.y = 0;
            if(valid)
                v = gload<C>(a.in, ibase, e, inverse);
            const unsigned long long u = lt_k1 * (unsigned long long)e;
            const T2 w = cmul(cmul(lt_tab[u & 255], lt_tab[256 + ((u >> 8) & 255)]), lt_tab[512 + ((u >> 16) & 255)]);
            return cmul(v, w);
        };
        auto g_dst = [&](int e, T2 v) {
            if(valid)
                gstore<C>(a.out, obase, e, v, inverse, use_sc, scale);
        };
        auto s_src = [=](int e) -> T2 { return sm[C::sidx(c, e)]; };
        auto s_dst = [=](int e, T2 v) { sm[C::sidx(c, e)] = v; };

        constexpr bool SI = C::CIN != COOP_NONE;
        constexpr bool SO = C::COUT != COOP_NONE;
        if constexpr(SI && SO)
            run_passes<C, 0, true, true>(t, c, sm, tw, s_src, s_dst);
        else if constexpr(SI)
            run_passes<C, 0, true, false>(t, c, sm, tw, s_src, g_dst);
        else if constexpr(SO)
        {
            if(LT_CAPABLE && lt_tab)
                run_passes<C, 0, false, true>(t, c, sm, tw, g_src_lt, s_dst);
            else
                run_passes<C, 0, false, true>(t, c, sm, tw, g_src, s_dst);
        }
        else
        {
            if(LT_CAPABLE && lt_tab)
                run_passes<C, 0, false, false>(t, c, sm, tw, g_src_lt, g_dst);
            else
                run_passes<C, 0, false, false>(t, c, sm, tw, g_src, g_dst);
        }

        // ---- cooperative store stage ----
        if constexpr(C::COUT == COOP_R2C_POST)
        {
            // shared memory holds Z = FFT_h of the packed real row (h = N); write
            // X_p = e + t d,  X_q = conj(e - t d),  e = (Z_p + conj Z_q)/2,
            // d = (Z_p - conj Z_q)/2,  t = -i W^p,  q = h - p.
            constexpr int H     = C::N;
            constexpr int NP    = H / 2 + 1;
            constexpr int ITEMS = NP * C::TPB;
            constexpr int ITER  = (ITEMS + C::THREADS - 1) / C::THREADS;
            const T2* __restrict__ htw = reinterpret_cast<const T2*>(a.aux[0]);
            const T sc = use_sc ? scale : (T)1;
#pragma unroll 4
            for(int it = 0; it < ITER; ++it)
            {
                const int idx = tid + it * C::THREADS;
                if(idx >= ITEMS)
                    break;
                const int cc = idx / NP;
                const int p  = idx % NP;
                const int q  = H - p;
                if((unsigned)cc >= nvalid)
                    continue;
                const long long ob = bases[2 * cc + 1];
                if(p == 0)
                {
                    const T2 z = sm[C::sidx(cc, 0)];
                    T2       x0, xh;
                    x0.x = (z.x + z.y) * sc;
                    x0.y = 0;
                    xh.x = (z.x - z.y) * sc;
                    xh.y = 0;
                    gstore<C>(a.out, ob, 0, x0, false, false, (T)1);
                    gstore<C>(a.out, ob, H, xh, false, false, (T)1);
                    continue;
                }
                const T2 za = sm[C::sidx(cc, p)];
                T2       zb = sm[C::sidx(cc, q)];
                zb.y        = -zb.y;
                const T2 w  = htw[p];
                T2       e, d, t;
                e.x = (za.x + zb.x) * (T)0.5;
                e.y = (za.y + zb.y) * (T)0.5;
                d.x = (za.x - zb.x) * (T)0.5;
                d.y = (za.y - zb.y) * (T)0.5;
                t.x = w.y; // -i * W^p
                t.y = -w.x;
                const T2 td = cmul(t, d);
                T2       xp, xq;
                xp.x = (e.x + td.x) * sc;
                xp.y = (e.y + td.y) * sc;
                xq.x = (e.x - td.x) * sc;
                xq.y = -(e.y - td.y) * sc;
                gstore<C>(a.out, ob, p, xp, false, false, (T)1);
                if(p != q)
                    gstore<C>(a.out, ob, q, xq, false, false, (T)1);
            }
        }
        else if constexpr(C::COUT != COOP_NONE)
        {
            // run_passes ended with a barrier because the last pass wrote shared memory
            for(int idx = tid; idx < C::N * C::TPB; idx += C::THREADS)
            {
                int cc, e;
                if constexpr(C::COUT == COOP_EFAST)
                {
                    cc = idx / C::N;
                    e  = idx % C::N;
                }
                else
                {
                    cc = idx % C::TPB;
                    e  = idx / C::TPB;
                }
                if((unsigned)cc < nvalid)
                    gstore<C>(a.out, bases[2 * cc + 1], e, sm[C::sidx(cc, e)], inverse, use_sc, scale);
            }
        }
    }

    // ------------------------------------------------------------------
    // Bluestein's algorithm for one tile, entirely in shared memory
    // ------------------------------------------------------------------
    // Transforms of arbitrary length n <= (M + 1) / 2 with M = C::N:
    //   a = x * chirp, zero padded to M;  A = FFT_M(a);  A *= filter;
    //   y = IFFT_M(A);  X_k = y_k * chirp_k          (chirp_p = exp(-i pi p^2 / n),
    //   filter = FFT_M(wrapped conj chirp) / M, both tables made on the host).
    // The chirp multiply rides on the first pass's global loads, the filter
    // multiply on the first pass of the second FFT and the final chirp
    // multiply on the last pass's global stores, so the kernel makes a single
    // HBM round trip over n points per transform.  The reference reaches this
    // form only up to M = 4096 (library/src/tree_node_bluestein.cpp:416-420);
    // 227 KB of shared memory per CTA carry it to M = 20480 in single precision.
    // kargs: iaux[0] = n, aux[0] = chirp (n entries), aux[1] = filter (M entries).
    template <class C>
    __global__ void __launch_bounds__(C::THREADS, C::MINB)
        bluestein_tile_kernel(const __grid_constant__ b200fft_kargs a)
    {
        using T  = typename C::T;
        using T2 = typename C::T2;
        extern __shared__ __align__(16) unsigned char smem_raw[];
        T2* sm = reinterpret_cast<T2*>(smem_raw);

        const int     tid     = threadIdx.x;
        const int     c       = tid / C::TPT;
        const int     t       = tid % C::TPT;
        const TilePos tp      = decode_tile(a, blockIdx.x, C::TPB);
        const bool    inverse = a.inverse != 0;
        const bool    use_sc  = a.use_scale != 0;
        const T       scale   = (T)a.scale;
        const int     n       = (int)a.iaux[0];
        const T2* __restrict__ tw    = reinterpret_cast<const T2*>(a.twiddles);
        const T2* __restrict__ chirp = reinterpret_cast<const T2*>(a.aux[0]);
        const T2* __restrict__ filt  = reinterpret_cast<const T2*>(a.aux[1]);

        const unsigned  nvalid = min((unsigned)C::TPB, a.on[0] - tp.i0_first);
        const bool      valid  = (unsigned)c < nvalid;
        // (slots past the last transform read the tile's first transform and discard it)
        const long long ibase  = view_base(a.in, tp.i0_first + (valid ? c : 0), tp.i1, tp.i2);
        const long long obase  = view_base(a.out, tp.i0_first + c, tp.i1, tp.i2);

        // branch-free (clamped index, result zeroed afterwards): with a branch around the load and the
        // multiply behind it the loads of a pass ran one after the other instead of back to back
        auto src1 = [&](int e) -> T2 {
            const int  ec   = min(e, n - 1);
            const T2   x    = gload<C>(a.in, ibase, ec, inverse);
            const T2   w    = chirp[ec];
            const bool live = valid && e < n;
            T2         v    = cmul(x, w);
            v.x             = live ? v.x : (T)0;
            v.y             = live ? v.y : (T)0;
            return v;
        };
        auto s_dst = [=](int e, T2 v) { sm[C::sidx(c, e)] = v; };
        run_passes<C, 0, false, true>(t, c, sm, tw, src1, s_dst);

        // second transform: inverse FFT as a forward FFT on exchanged parts
        auto src2 = [=](int e) -> T2 { return cswap(cmul(sm[C::sidx(c, e)], filt[e])); };
        auto dst2 = [&](int e, T2 v) {
            if(valid && e < n)
                gstore<C>(a.out, obase, e, cmul(cswap(v), chirp[e]), inverse, use_sc, scale);
        };
        run_passes<C, 0, true, false>(t, c, sm, tw, src2, dst2);
    }

    template <class C>
    cudaError_t launch_bluestein_kernel(const b200fft_kargs& a, unsigned long long ntiles, cudaStream_t stream)
    {
        static std::atomic<bool> attr_done[64]; // zero-initialised; host threads may launch the same kernel concurrently
        int         dev           = 0;
        cudaGetDevice(&dev);
        if(C::SMEM_BYTES > 48 * 1024 && dev < 64 && !attr_done[dev])
        {
            cudaError_t e = cudaFuncSetAttribute(bluestein_tile_kernel<C>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)C::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            attr_done[dev] = true;
        }
        if(ntiles == 0)
            return cudaSuccess;
        if(ntiles > 0x7fffffffull)
            return cudaErrorInvalidConfiguration;
        bluestein_tile_kernel<C><<<(unsigned)ntiles, C::THREADS, C::SMEM_BYTES, stream>>>(a);
        return cudaGetLastError();
    }

    // host-side launch helper used by generated launchers
    template <class C>
    cudaError_t launch_tile_kernel(const b200fft_kargs& a, unsigned long long ntiles, cudaStream_t stream)
    {
        static std::atomic<bool> attr_done[64]; // zero-initialised; host threads may launch the same kernel concurrently
        int         dev           = 0;
        cudaGetDevice(&dev);
        if(C::SMEM_BYTES > 48 * 1024 && dev < 64 && !attr_done[dev])
        {
            cudaError_t e = cudaFuncSetAttribute(stockham_tile_kernel<C>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)C::SMEM_BYTES);
            if(e != cudaSuccess)
                return e;
            attr_done[dev] = true;
        }
        if(ntiles == 0)
            return cudaSuccess;
        if(ntiles > 0x7fffffffull)
            return cudaErrorInvalidConfiguration;
        stockham_tile_kernel<C><<<(unsigned)ntiles, C::THREADS, C::SMEM_BYTES, stream>>>(a);
        return cudaGetLastError();
    }
} // namespace b200fft
