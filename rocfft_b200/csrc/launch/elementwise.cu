// Element-wise helper kernels: layout copies, real <-> Hermitian conversions,
// even-length real pre/post-processing, Bluestein multiplies and the large-1D
// twiddle multiply.  They are the general (any stride, planar or interleaved)
// building blocks; the fused Stockham kernels replace them on the fast paths.
//
// Roles in the reference:
//   copies ................ library/src/rtc_realcomplex_gen.cpp:63-298
//                           (r2c_copy, c2r_copy, c2herm_copy, herm2c_copy)
//   real pre/post ......... library/src/rtc_realcomplex_gen.cpp:348-573,
//                           device/kernels/real2complex_device.h:25-254
//   Bluestein multiplies .. library/src/rtc_bluestein_gen.cpp:170-396
//   large twiddles ........ device/kernels/common.h:227-301
//
// One thread handles one point (or one conjugate pair) of one transform; the
// grid is a flat grid-stride loop over points x transforms.
#include "launch.h"
#include "../kernels/stockham_engine.cuh"

namespace b200fft
{
    template <typename T>
    struct EwIo
    {
        using T2 = typename cx<T>::type;
        static __device__ __forceinline__ T2 loadc(const b200fft_ioview& v, long long off)
        {
            T2 r;
            if(v.planar)
            {
                r.x = reinterpret_cast<const T*>(v.p[0])[off];
                r.y = reinterpret_cast<const T*>(v.p[1])[off];
            }
            else
                r = reinterpret_cast<const T2*>(v.p[0])[off];
            return r;
        }
        static __device__ __forceinline__ void storec(const b200fft_ioview& v, long long off, T2 val)
        {
            if(v.planar)
            {
                reinterpret_cast<T*>(v.p[0])[off] = val.x;
                reinterpret_cast<T*>(v.p[1])[off] = val.y;
            }
            else
                reinterpret_cast<T2*>(v.p[0])[off] = val;
        }
    };

    template <typename T, int KIND>
    __global__ void __launch_bounds__(256) elementwise_kernel(const __grid_constant__ b200fft_eargs a)
    {
        using T2 = typename cx<T>::type;
        using IO = EwIo<T>;

        // number of work items per transform
        unsigned work;
        if(KIND == B200FFT_EW_R2C_POST || KIND == B200FFT_EW_C2R_PRE)
            work = a.n / 2 + 1; // a.n = half length h; pairs p = 0..h/2
        else if(KIND == B200FFT_EW_BLUE_PAD_MUL || KIND == B200FFT_EW_HERM2C_COPY)
            work = (unsigned)a.iaux[0]; // padded / full length
        else
            work = a.n;

        const unsigned long long ntrans = (unsigned long long)a.on[0] * a.on[1] * a.on[2];
        const unsigned long long total  = ntrans * work;
        const bool               inv    = a.inverse != 0;
        const T                  sc     = a.use_scale ? (T)a.scale : (T)1;

        for(unsigned long long idx = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
            idx += (unsigned long long)gridDim.x * blockDim.x)
        {
            const unsigned     p  = (unsigned)(idx % work);
            unsigned long long r  = idx / work;
            const unsigned     i0 = (unsigned)(r % a.on[0]);
            r /= a.on[0];
            const unsigned  i1 = (unsigned)(r % a.on[1]);
            const unsigned  i2 = (unsigned)(r / a.on[1]);
            const long long ib = view_base(a.in, i0, i1, i2);
            const long long ob = view_base(a.out, i0, i1, i2);

            if constexpr(KIND == B200FFT_EW_COPY_C2C)
            {
                T2 v = IO::loadc(a.in, ib + (long long)p * a.in.es);
                v.x *= sc;
                v.y *= sc;
                IO::storec(a.out, ob + (long long)p * a.out.es, v);
            }
            else if constexpr(KIND == B200FFT_EW_R2C_COPY)
            {
                T2 v;
                v.x = reinterpret_cast<const T*>(a.in.p[0])[ib + (long long)p * a.in.es];
                v.y = 0;
                IO::storec(a.out, ob + (long long)p * a.out.es, v);
            }
            else if constexpr(KIND == B200FFT_EW_C2R_COPY)
            {
                // a transform computed with swapped parts leaves its real result in .y
                T2 v = IO::loadc(a.in, ib + (long long)p * a.in.es);
                reinterpret_cast<T*>(a.out.p[0])[ob + (long long)p * a.out.es] = (inv ? v.y : v.x) * sc;
            }
            else if constexpr(KIND == B200FFT_EW_HERM2C_COPY)
            {
                // full length N = iaux[0]; input holds points 0..N/2
                const unsigned N = (unsigned)a.iaux[0];
                T2             v;
                if(p <= N / 2)
                {
                    v = IO::loadc(a.in, ib + (long long)p * a.in.es);
                    if(p == 0 || 2 * p == N)
                        v.y = 0; // the imaginary parts of DC and Nyquist carry no information
                }
                else
                {
                    v   = IO::loadc(a.in, ib + (long long)(N - p) * a.in.es);
                    v.y = -v.y;
                }
                if(inv)
                    v = cswap(v);
                IO::storec(a.out, ob + (long long)p * a.out.es, v);
            }
            else if constexpr(KIND == B200FFT_EW_R2C_POST)
            {
                // in: Z = FFT_h of the packed real row; out: X[0..h]
                const unsigned h = a.n;
                const unsigned q = h - p;
                if(p > q)
                    continue;
                const T2* __restrict__ tw = reinterpret_cast<const T2*>(a.aux[0]); // exp(-2 pi i p / 2h)
                if(p == 0)
                {
                    T2 z = IO::loadc(a.in, ib);
                    T2 x0, xh;
                    x0.x = (z.x + z.y) * sc;
                    x0.y = 0;
                    xh.x = (z.x - z.y) * sc;
                    xh.y = 0;
                    IO::storec(a.out, ob, x0);
                    IO::storec(a.out, ob + (long long)h * a.out.es, xh);
                }
                else
                {
                    T2 za = IO::loadc(a.in, ib + (long long)p * a.in.es);
                    T2 zb = IO::loadc(a.in, ib + (long long)q * a.in.es);
                    zb.y  = -zb.y;
                    T2 e, d, t, w = tw[p];
                    e.x = (za.x + zb.x) * (T)0.5;
                    e.y = (za.y + zb.y) * (T)0.5;
                    d.x = (za.x - zb.x) * (T)0.5;
                    d.y = (za.y - zb.y) * (T)0.5;
                    t.x = w.y; // -i * W^p
                    t.y = -w.x;
                    T2 td = cmul(t, d);
                    T2 xp, xq;
                    xp.x = (e.x + td.x) * sc;
                    xp.y = (e.y + td.y) * sc;
                    xq.x = (e.x - td.x) * sc;
                    xq.y = -(e.y - td.y) * sc;
                    IO::storec(a.out, ob + (long long)p * a.out.es, xp);
                    if(p != q)
                        IO::storec(a.out, ob + (long long)q * a.out.es, xq);
                }
            }
            else if constexpr(KIND == B200FFT_EW_C2R_PRE)
            {
                // in: X[0..h]; out: Z' (h points) whose unnormalised inverse FFT_h is the
                // packed real row (even samples in the real parts, odd in the imaginary).
                const unsigned h = a.n;
                const unsigned q = h - p;
                if(p > q)
                    continue;
                const T2* __restrict__ tw = reinterpret_cast<const T2*>(a.aux[0]);
                T2 xa = IO::loadc(a.in, ib + (long long)p * a.in.es);
                T2 xb = IO::loadc(a.in, ib + (long long)q * a.in.es);
                if(p == 0)
                {
                    xa.y = 0;
                    xb.y = 0;
                }
                xb.y = -xb.y;
                T2 e, d, t, w = tw[p];
                e.x = xa.x + xb.x;
                e.y = xa.y + xb.y;
                d.x = xa.x - xb.x;
                d.y = xa.y - xb.y;
                t.x = w.y; // i * conj(W^p)
                t.y = w.x;
                T2 td = cmul(t, d);
                T2 zp, zq;
                zp.x = e.x + td.x;
                zp.y = e.y + td.y;
                zq.x = e.x - td.x;
                zq.y = -(e.y - td.y);
                IO::storec(a.out, ob + (long long)p * a.out.es, zp);
                if(p != q && p != 0)
                    IO::storec(a.out, ob + (long long)q * a.out.es, zq);
            }
            else if constexpr(KIND == B200FFT_EW_BLUE_PAD_MUL)
            {
                const T2* __restrict__ chirp = reinterpret_cast<const T2*>(a.aux[0]);
                T2 v;
                v.x = 0;
                v.y = 0;
                if(p < a.n)
                {
                    v = IO::loadc(a.in, ib + (long long)p * a.in.es);
                    if(inv)
                        v = cswap(v);
                    v = cmul(v, chirp[p]);
                }
                IO::storec(a.out, ob + (long long)p * a.out.es, v);
            }
            else if constexpr(KIND == B200FFT_EW_POINT_MUL)
            {
                const T2* __restrict__ tab = reinterpret_cast<const T2*>(a.aux[0]);
                T2 v = IO::loadc(a.in, ib + (long long)p * a.in.es);
                IO::storec(a.out, ob + (long long)p * a.out.es, cmul(v, tab[p]));
            }
            else if constexpr(KIND == B200FFT_EW_BLUE_RES_MUL)
            {
                const T2* __restrict__ chirp = reinterpret_cast<const T2*>(a.aux[0]);
                T2 v = cmul(IO::loadc(a.in, ib + (long long)p * a.in.es), chirp[p]);
                if(inv)
                    v = cswap(v);
                v.x *= sc;
                v.y *= sc;
                IO::storec(a.out, ob + (long long)p * a.out.es, v);
            }
            else if constexpr(KIND == B200FFT_EW_LARGE_TWIDDLE)
            {
                // rows of n = n1*n2 points laid out [k1][i2]; iaux[0] = n2, iaux[1] = table steps
                const unsigned n2 = (unsigned)a.iaux[0];
                const unsigned k1 = p / n2, i2 = p % n2;
                const T2*      tab = reinterpret_cast<const T2*>(a.aux[0]);
                T2 w = large_twiddle(tab, (unsigned long long)k1 * i2, (int)a.iaux[1]);
                if(inv)
                    w.y = -w.y; // an inverse transform runs on exchanged parts: use the conjugate
                T2 v = IO::loadc(a.in, ib + (long long)p * a.in.es);
                IO::storec(a.out, ob + (long long)p * a.out.es, cmul(v, w));
            }
        }
    }

    // ------------------------------------------------------------------
    // tiled transposing copy
    // ------------------------------------------------------------------
    // Role in the reference: the out-of-place tiled transpose kernel, library/src/rtc_transpose_gen.cpp:77-326
    // (64 x 64 tiles through LDS, launch shapes library/src/rtc_transpose_kernel.cpp:40-75).  The N-D plans
    // here need no transposes, but a layout change whose fastest dimension differs between input and output
    // (an in-place transform with transposed output strides, for one) is a transpose all the same: the flat
    // copy above would read lines and write single points.  This kernel moves 32 x 32 tiles through padded
    // shared memory so that both the reads (along dimension DA, unit input stride) and the writes (along
    // DB, unit output stride) are coalesced; the two remaining dimensions are walked by the grid.
    // The index space has four dimensions: 0 = the points of a transform (n, es), 1..3 = on[0..2] (os[0..2]).
    struct TransposeDims
    {
        unsigned  len[4];
        long long is[4], os[4];
        int       da, db, dc, dd;
        unsigned  ta, tb; // tiles along DA / DB
    };

    template <typename T>
    __global__ void __launch_bounds__(256) transpose_tile_kernel(const __grid_constant__ b200fft_eargs a,
                                                                  const __grid_constant__ TransposeDims d)
    {
        using T2 = typename cx<T>::type;
        __shared__ T2 tile[32][33];
        unsigned long long blk = blockIdx.x;
        const unsigned     ta  = (unsigned)(blk % d.ta);
        blk /= d.ta;
        const unsigned tb = (unsigned)(blk % d.tb);
        blk /= d.tb;
        const unsigned  ic = (unsigned)(blk % d.len[d.dc]);
        const unsigned  id = (unsigned)(blk / d.len[d.dc]);
        const long long ibase = (long long)ic * d.is[d.dc] + (long long)id * d.is[d.dd];
        const long long obase = (long long)ic * d.os[d.dc] + (long long)id * d.os[d.dd];
        const T         sc    = a.use_scale ? (T)a.scale : (T)1;
        const T2*       in    = reinterpret_cast<const T2*>(a.in.p[0]);
        T2*             out   = reinterpret_cast<T2*>(a.out.p[0]);
        const unsigned  tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
        {
            const unsigned ia = ta * 32 + tx;
#pragma unroll
            for(unsigned r = ty; r < 32; r += 8)
            {
                const unsigned ib = tb * 32 + r;
                if(ia < d.len[d.da] && ib < d.len[d.db])
                    tile[r][tx] = in[ibase + (long long)ia * d.is[d.da] + (long long)ib * d.is[d.db]];
            }
        }
        __syncthreads();
        {
            const unsigned ib = tb * 32 + tx;
#pragma unroll
            for(unsigned r = ty; r < 32; r += 8)
            {
                const unsigned ia = ta * 32 + r;
                if(ia < d.len[d.da] && ib < d.len[d.db])
                {
                    T2 v = tile[tx][r];
                    v.x *= sc;
                    v.y *= sc;
                    out[obase + (long long)ia * d.os[d.da] + (long long)ib * d.os[d.db]] = v;
                }
            }
        }
    }

    // true when the copy is a transpose this kernel serves; fills `d`
    inline bool transpose_shape(const b200fft_eargs& a, TransposeDims& d)
    {
        if(a.in.planar || a.out.planar)
            return false;
        d.len[0] = a.n;
        d.is[0]  = a.in.es;
        d.os[0]  = a.out.es;
        for(int k = 0; k < 3; ++k)
        {
            d.len[k + 1] = a.on[k];
            d.is[k + 1]  = a.in.os[k];
            d.os[k + 1]  = a.out.os[k];
        }
        d.da = d.db = -1;
        for(int k = 0; k < 4; ++k)
        {
            if(d.len[k] < 16)
                continue;
            if(d.is[k] == 1 && (d.da < 0 || d.len[k] > d.len[d.da]))
                d.da = k;
            if(d.os[k] == 1 && (d.db < 0 || d.len[k] > d.len[d.db]))
                d.db = k;
        }
        if(d.da < 0 || d.db < 0 || d.da == d.db)
            return false; // same fastest dimension on both sides (or none): the flat copy is already coalesced
        d.dc = d.dd = -1;
        for(int k = 0; k < 4; ++k)
            if(k != d.da && k != d.db)
                (d.dc < 0 ? d.dc : d.dd) = k;
        d.ta = (d.len[d.da] + 31) / 32;
        d.tb = (d.len[d.db] + 31) / 32;
        const unsigned long long blocks = (unsigned long long)d.ta * d.tb * d.len[d.dc] * d.len[d.dd];
        return blocks > 0 && blocks <= 0x7fffffffull;
    }

    template <typename T, int KIND>
    cudaError_t launch_ew(const b200fft_eargs& a, cudaStream_t stream)
    {
        if constexpr(KIND == B200FFT_EW_COPY_C2C)
        {
            TransposeDims d;
            if(a.on[0] && a.on[1] && a.on[2] && a.n && transpose_shape(a, d))
            {
                const unsigned long long blocks = (unsigned long long)d.ta * d.tb * d.len[d.dc] * d.len[d.dd];
                transpose_tile_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(a, d);
                return cudaGetLastError();
            }
        }
        unsigned work;
        if(KIND == B200FFT_EW_R2C_POST || KIND == B200FFT_EW_C2R_PRE)
            work = a.n / 2 + 1;
        else if(KIND == B200FFT_EW_BLUE_PAD_MUL || KIND == B200FFT_EW_HERM2C_COPY)
            work = (unsigned)a.iaux[0];
        else
            work = a.n;
        const unsigned long long total = (unsigned long long)a.on[0] * a.on[1] * a.on[2] * work;
        if(total == 0)
            return cudaSuccess;
        unsigned long long blocks = (total + 255) / 256;
        if(blocks > 148ull * 64)
            blocks = 148ull * 64;
        elementwise_kernel<T, KIND><<<(unsigned)blocks, 256, 0, stream>>>(a);
        return cudaGetLastError();
    }

    template <typename T>
    cudaError_t dispatch_ew(int kind, const b200fft_eargs& a, cudaStream_t s)
    {
        switch(kind)
        {
        case B200FFT_EW_COPY_C2C:
        case B200FFT_EW_C2HERM_COPY:
            return launch_ew<T, B200FFT_EW_COPY_C2C>(a, s);
        case B200FFT_EW_R2C_COPY:
            return launch_ew<T, B200FFT_EW_R2C_COPY>(a, s);
        case B200FFT_EW_C2R_COPY:
            return launch_ew<T, B200FFT_EW_C2R_COPY>(a, s);
        case B200FFT_EW_HERM2C_COPY:
            return launch_ew<T, B200FFT_EW_HERM2C_COPY>(a, s);
        case B200FFT_EW_R2C_POST:
            return launch_ew<T, B200FFT_EW_R2C_POST>(a, s);
        case B200FFT_EW_C2R_PRE:
            return launch_ew<T, B200FFT_EW_C2R_PRE>(a, s);
        case B200FFT_EW_BLUE_PAD_MUL:
            return launch_ew<T, B200FFT_EW_BLUE_PAD_MUL>(a, s);
        case B200FFT_EW_POINT_MUL:
            return launch_ew<T, B200FFT_EW_POINT_MUL>(a, s);
        case B200FFT_EW_BLUE_RES_MUL:
            return launch_ew<T, B200FFT_EW_BLUE_RES_MUL>(a, s);
        case B200FFT_EW_LARGE_TWIDDLE:
            return launch_ew<T, B200FFT_EW_LARGE_TWIDDLE>(a, s);
        default:
            return cudaErrorInvalidValue;
        }
    }
} // namespace b200fft

// ---- buffer hash for the kernelio log layer ----
// Order-independent 64-bit checksum of a byte range: every 8-byte word is mixed with its index and the
// results are summed (the reference's kernelio layer hashes each kernel's input and output,
// library/src/powX.cpp:743-780, 910-956; this serves the same purpose: telling, kernel by kernel, whether
// two runs saw the same data).
namespace b200fft
{
    static __global__ void __launch_bounds__(256) hash_words_kernel(const unsigned long long* p, size_t words, unsigned long long* out)
    {
        unsigned long long acc = 0;
        for(size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (size_t)gridDim.x * blockDim.x)
        {
            unsigned long long v = p[i] ^ (0x9E3779B97F4A7C15ull * (unsigned long long)(i + 1));
            v ^= v >> 31;
            v *= 0xBF58476D1CE4E5B9ull;
            v ^= v >> 29;
            acc += v;
        }
        for(int o = 16; o > 0; o >>= 1)
            acc += __shfl_down_sync(0xffffffffu, acc, o);
        if((threadIdx.x & 31) == 0)
            atomicAdd(out, acc);
    }
}

extern "C" cudaError_t b200fft_launch_hash(const void* p, size_t bytes, unsigned long long* out, cudaStream_t stream)
{
    const size_t words = bytes / 8;
    if(cudaMemsetAsync(out, 0, sizeof(unsigned long long), stream) != cudaSuccess)
        return cudaGetLastError();
    if(words == 0)
        return cudaSuccess;
    size_t blocks = (words + 255) / 256;
    if(blocks > 148 * 16)
        blocks = 148 * 16;
    b200fft::hash_words_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const unsigned long long*>(p), words, out);
    return cudaGetLastError();
}

extern "C" cudaError_t
    b200fft_launch_elementwise(int kind, int precision, const b200fft_eargs* a, cudaStream_t stream)
{
    if(precision == 0)
        return b200fft::dispatch_ew<float>(kind, *a, stream);
    return b200fft::dispatch_ew<double>(kind, *a, stream);
}
