// Whole 2D transforms of N x N images in ONE persistent kernel whose intermediate
// array never leaves the L2 cache.
//
// Role in the reference: the 2D plans RTRT / RC (library/src/tree_node_2D.cpp:31-211,
// row FFTs, transposes or a fused row/column pair, column FFTs) make two to four trips
// through device memory per image.  B200's L2 (126 MB) holds several 1024 x 1024 images,
// so here the row pass of image k and the column pass of image k-D (D = 1 to 3) are interleaved in one
// launch: the rows of an image are read from HBM, transformed and written back (the lines
// stay dirty in L2), and a short while later the column tiles of the same image are read
// back — from L2 — transformed and written for good.  Per image the device memory sees one
// read and one write: the algorithmic minimum.  A 3D transform uses the kernel for its XY
// planes and makes one more pass for Z.
//
// Work list.  Item i belongs to block k = i / (TR + TC): the first TR items of a block are
// the row tiles of image k, the remaining TC items the column tiles of image k-D (the first D
// blocks have no column part, the last D no row part; D is chosen by the launcher: 1 in double
// precision, 3 in single, from measurements).  CTA c takes items c, c + G, c + 2G, ...
// in order.  A column tile may only be loaded once all TR row tiles of its image are
// stored: every CTA that finishes a row tile makes its stores visible (fence) and adds one
// to the image's counter; the thread that issues a column tile's loads first waits — with a
// bound — for the counter to reach TR.  Dependencies point to earlier items only and row
// tiles never wait, so the list always makes progress as long as all CTAs are resident,
// which the cooperative launch guarantees.
//
// A CTA's pipeline is that of the column kernel (stockham_colstream.cuh): one shared-memory
// stage filled by the copy engines (bulk copies of whole rows for a row tile, tensor-copy
// boxes for a column tile) on an mbarrier; every thread moves its points into registers,
// the stage is refilled for the NEXT item at once, and the two radix passes run out of
// registers with one exchange through shared memory in between (inside a warp for row
// tiles: the 32 lanes of a warp hold one row — or one pair of rows in packed single
// precision — so the exchange needs no CTA barrier).
//
// Requirements (planner): square power-of-two images with two radix passes (N = 1024:
// 32 x 32), interleaved complex, unit stride along rows, rows back to back, 16-byte aligned
// bases, image strides multiples of 16 bytes.
#pragma once
#include "stockham_colstream.cuh"

namespace b200fft
{
    namespace ptx
    {
        __device__ __forceinline__ int ld_acquire_gpu(const int* p)
        {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
            return v;
        }
        // orders generic-proxy observations before the async-proxy (copy engine) accesses that follow
        __device__ __forceinline__ void fence_proxy_async_all()
        {
            asm volatile("fence.proxy.async;" ::: "memory");
        }
    }

#ifndef B200FFT_DEP_SPIN
#define B200FFT_DEP_SPIN (1u << 24) // polls of an image's row counter before a wait gives up
#endif

    template <class C, int UN>
    struct FusedL2
    {
        // single precision in scalar form (one column per thread, 16 warps per 128-byte-wide tile)
        static constexpr bool SC         = sizeof(typename C::T) == 4;
        using CC                         = ColStream<C, UN, SC>;
        using T                          = typename C::T;
        using T2                         = typename C::T2;
        static constexpr int N           = C::N;
        static constexpr int VEC         = CC::VEC;
        static constexpr int THREADS     = CC::THREADS; // 32 lanes x UN
        static constexpr int WARPS       = THREADS / 32;
        static constexpr int ROWS        = WARPS * VEC; // rows of a row tile
        static constexpr int TR          = N / ROWS; // row tiles per image
        static constexpr int TC          = N / CC::COLS; // column tiles per image
        static constexpr size_t SMEM_BYTES = CC::SMEM_BYTES;
        static_assert(C::TPT == 32 && C::NPASS == 2 && CC::EPT == 32, "two radix-32-wide passes, one butterfly per lane");
        static_assert((unsigned)ROWS * N * sizeof(T2) == CC::STAGE_BYTES, "row tiles and column tiles share the stage");
        static_assert(CC::OBOX_ROWS == CC::BOX_ROWS, "loads and stores of column tiles use one tensor map");
    };

    // kargs: in / out = the images (p[0], os[1] = image stride in elements; rows back to back),
    // on[1] = number of images, twiddles = stacked table of the N-point transform,
    // aux[1] = int counters, one per image, zero at launch; aux[3] = device error flag.
    // `map` = tensor map of the OUTPUT array (dimension 0 columns in 8-byte elements, then the
    // dimensions ordered as iaux[3] says, see stockham_colstream.cuh).
    template <class C, int UN>
    __global__ void __launch_bounds__(FusedL2<C, UN>::THREADS, C::MINB)
        stockham_fused2d_kernel(const __grid_constant__ b200fft_kargs a, const __grid_constant__ CUtensorMap map)
    {
        using F  = FusedL2<C, UN>;
        using CC = typename F::CC;
        using T  = typename C::T;
        using T2 = typename C::T2;
        using U  = typename CC::U;
        using C2 = typename CC::C2;
        using PV = typename CC::P;
        using SV = typename CC::SV;
        constexpr int N = C::N;
        extern __shared__ unsigned char smem_dyn[];
        unsigned char* smem_raw = smem_dyn + ((256u - (ptx::smem_u32(smem_dyn) & 255u)) & 255u);
        U*             stage    = reinterpret_cast<U*>(smem_raw);
        PV*            xs       = reinterpret_cast<PV*>(smem_raw + CC::STAGE_BYTES);
        uint64_t*      full     = reinterpret_cast<uint64_t*>(smem_raw + CC::STAGE_BYTES + CC::XCHG_BYTES);

        const int tid  = threadIdx.x;
        const int lane = tid & 31;
        const int warp = tid >> 5;
        const T2* __restrict__ tw = reinterpret_cast<const T2*>(a.twiddles);
        const T sgn = a.inverse ? (T)-1 : (T)1;
        const T sx  = a.use_scale ? (T)a.scale : (T)1;
        const T sy  = sx * sgn;
        int*    err  = reinterpret_cast<int*>(const_cast<void*>(a.aux[3]));
        int*    done = reinterpret_cast<int*>(const_cast<void*>(a.aux[1]));
        const unsigned nimg = a.on[1];
        constexpr unsigned B = F::TR + F::TC;
        // column tiles run D images behind the row tiles
        const unsigned D = (unsigned)a.iaux[2];
        const unsigned long long nitems = (unsigned long long)(nimg + D) * B;
        const int pe = (int)(a.iaux[3] & 3), p1 = (int)((a.iaux[3] >> 2) & 3);

        // twiddles of the second pass in shared memory (both tile kinds use the same 32 x 32 table)
        typename SV::TWS* tws = reinterpret_cast<typename SV::TWS*>(smem_raw + CC::STAGE_BYTES + CC::XCHG_BYTES + 16);
        for(int i = tid; i < CC::TW_ENTRIES; i += F::THREADS)
            tws[i] = SV::tws(tw[i]);
        if(tid == 0)
        {
            ptx::mbar_init(full, 1);
            ptx::fence_mbar_init();
        }
        __syncthreads();

        // item -> (kind, image, tile); items of the half-empty first and last blocks are skipped
        auto valid_from = [&](unsigned long long i) -> unsigned long long {
            for(; i < nitems; i += gridDim.x)
            {
                const unsigned k = (unsigned)(i / B), off = (unsigned)(i % B);
                if(off < (unsigned)F::TR ? k < nimg : k >= D)
                    return i;
            }
            return nitems;
        };
        // thread 0 only.  Returns false when the item's rows are not stored yet (`poll` bounded).
        auto try_issue = [&](unsigned long long i, unsigned polls) -> bool {
            const unsigned k = (unsigned)(i / B), off = (unsigned)(i % B);
            if(off < (unsigned)F::TR)
            {
                // row tile: ROWS whole rows of image k, one contiguous range of the input
                const unsigned char* src = reinterpret_cast<const unsigned char*>(
                    reinterpret_cast<const T2*>(a.in.p[0]) + (long long)k * a.in.os[1] + (long long)off * F::ROWS * N);
                ptx::mbar_expect_tx(full, CC::STAGE_BYTES + B200FFT_TEST_EXTRA_TX);
                constexpr unsigned CHUNK = CC::STAGE_BYTES / 4;
#pragma unroll
                for(int q = 0; q < 4; ++q)
                    ptx::bulk_load(reinterpret_cast<unsigned char*>(stage) + q * CHUNK, src + q * CHUNK, CHUNK, full);
                return true;
            }
            const unsigned img = k - D, tile = off - F::TR;
            bool ready = false;
            for(unsigned p = 0; p < polls && !ready; ++p)
                ready = ptx::ld_acquire_gpu(done + img) >= F::TR;
            if(!ready)
                return false;
            ptx::fence_proxy_async_all(); // the rows were written through the generic proxy; the copy engine reads them
            ptx::mbar_expect_tx(full, CC::STAGE_BYTES + B200FFT_TEST_EXTRA_TX);
#pragma unroll
            for(int bx = 0; bx < CC::NBOX; ++bx)
            {
                const int row = bx * CC::BOX_ROWS;
                const int c1  = pe == 0 ? row : (p1 == 0 ? (int)img : 0);
                const int c2  = pe == 1 ? row : (p1 == 1 ? (int)img : 0);
                const int c3  = pe == 2 ? row : (p1 == 2 ? (int)img : 0);
                ptx::tma_load_4d(reinterpret_cast<unsigned char*>(stage) + (size_t)bx * CC::BOX_ROWS * CC::ROW_BYTES,
                                 &map,
                                 (int)(tile * (unsigned)CC::COLS * (unsigned)(sizeof(T2) / 8)),
                                 c1,
                                 c2,
                                 c3,
                                 full);
            }
            return true;
        };
        __shared__ int s_abort, s_deferred;
        if(tid == 0)
            s_abort = s_deferred = 0;

        unsigned long long cur = valid_from(blockIdx.x);
        if(tid == 0 && cur < nitems)
        {
            if(!try_issue(cur, B200FFT_DEP_SPIN))
            {
                if(err)
                    atomicExch(err, 1);
                s_abort = 1;
            }
        }
        __syncthreads();
        unsigned phase = 0;
        while(cur < nitems)
        {
            if(s_abort)
                break;
            const unsigned k = (unsigned)(cur / B), off = (unsigned)(cur % B);
            const bool     is_rows = off < (unsigned)F::TR;
            const bool     landed  = ptx::mbar_wait(full, phase);
            phase ^= 1u;
            if(tid == 0)
                ptx::bulk_wait_read<0>(); // tensor stores of an earlier column tile have read the exchange buffer
            C2 r[32];
            if(landed)
            {
                if(is_rows)
                {
                    // lane t of warp w: points t + 32 j of row(s) VEC * w (+1)
                    const T2* rows = reinterpret_cast<const T2*>(stage) + (size_t)warp * F::VEC * N;
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                    {
                        if constexpr(F::VEC == 2)
                        {
                            const float2 p0 = rows[lane + 32 * j], p1v = rows[N + lane + 32 * j];
                            r[j].x = pk2(p0.x, p1v.x);
                            r[j].y = pk2(p0.y * sgn, p1v.y * sgn);
                        }
                        else
                        {
                            const T2 p0 = rows[lane + 32 * j];
                            r[j].x      = p0.x;
                            r[j].y      = p0.y * sgn;
                        }
                    }
                }
                else
                {
                    const int u = tid % CC::UNITS, tl = tid / CC::UNITS;
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                        r[j] = SV::unpack(stage[(tl + j * 32) * CC::UNITS + u], (T)1);
                }
            }
            if(__syncthreads_or(landed ? 0 : 1))
            {
                if(tid == 0)
                {
                    if(err)
                        atomicExch(err, 1);
                    ptx::mbar_wait(full, phase ^ 1u);
                    ptx::bulk_wait_all(); // our own stores
                }
                __syncthreads();
                return;
            }
            // the stage is free: start the copy of the next item unless its rows are still being written
            // (thread 0 notes a deferral in shared memory; everybody reads it after the barriers of the passes)
            const unsigned long long nxt = valid_from(cur + gridDim.x);
            if(tid == 0)
                s_deferred = (nxt < nitems && !try_issue(nxt, 1)) ? 1 : 0;

            if(is_rows)
            {
                // ---- row tile: both passes inside the warp ----
                Butterfly<32, C2>::run(r);
                PV* xw = xs + (size_t)warp * CC::XROWS; // this warp's part of the exchange buffer
#pragma unroll
                for(int half = 0; half < 2; ++half)
                {
                    __syncwarp();
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                        xw[CC::prow(32 * lane + j)] = half == 0 ? r[j].x : r[j].y;
                    __syncwarp();
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                    {
                        const PV v = xw[CC::prow(lane + 32 * j)];
                        if(half == 0)
                            r[j].x = v;
                        else
                            r[j].y = v;
                    }
                }
#pragma unroll
                for(int j = 1; j < 32; ++j)
                    r[j] = SV::twmul(r[j], tws[(j - 1) * 32 + lane]);
                Butterfly<32, C2>::run(r);
                // results: points lane + 32 j of the row(s); the conjugation of an inverse transform
                // is undone after the column pass only, the scale factor is applied there as well
                T2* orow = reinterpret_cast<T2*>(a.out.p[0]) + (long long)k * a.out.os[1]
                           + ((long long)off * F::ROWS + (long long)warp * F::VEC) * N;
#pragma unroll
                for(int j = 0; j < 32; ++j)
                {
                    if constexpr(F::VEC == 2)
                    {
                        orow[lane + 32 * j]     = make_float2(r[j].x.v.x, r[j].y.v.x);
                        orow[N + lane + 32 * j] = make_float2(r[j].x.v.y, r[j].y.v.y);
                    }
                    else
                    {
                        T2 o;
                        o.x                 = r[j].x;
                        o.y                 = r[j].y;
                        orow[lane + 32 * j] = o;
                    }
                }
                // publish: every thread's stores before the counter moves
                __threadfence();
                __syncthreads();
                if(tid == 0)
                    atomicAdd(done + k, 1);
            }
            else
            {
                // ---- column tile of image k-D: as in the column kernel ----
                // (results leave as tensor stores through the exchange buffer)
                const unsigned img = k - D, tile = off - F::TR;
                const int      u = tid % CC::UNITS, tl = tid / CC::UNITS;
                colstream_run<CC, 0>(r, xs, tws, tl, u);
                colstream_store_staged<CC>(r, xs, tl, u, tid, sx, sy, [&](int row, const unsigned char* src) {
                    const int c1 = pe == 0 ? row : (p1 == 0 ? (int)img : 0);
                    const int c2 = pe == 1 ? row : (p1 == 1 ? (int)img : 0);
                    const int c3 = pe == 2 ? row : (p1 == 2 ? (int)img : 0);
                    ptx::tma_store_4d(&map, (int)(tile * (unsigned)CC::COLS * (unsigned)(sizeof(T2) / 8)), c1, c2, c3, src);
                });
            }
            if(s_deferred)
            {
                if(tid == 0 && !try_issue(nxt, B200FFT_DEP_SPIN))
                {
                    if(err)
                        atomicExch(err, 1);
                    s_abort = 1;
                }
                __syncthreads();
            }
            cur = nxt;
        }
        if(tid == 0)
            ptx::bulk_wait_all(); // nothing of ours may be in flight when the CTA retires
    }

    template <class C, int UN>
    cudaError_t launch_fused2d_kernel(const b200fft_kargs& a, unsigned long long nimages, cudaStream_t stream)
    {
        using F  = FusedL2<C, UN>;
        using CC = typename F::CC;
        using T2 = typename C::T2;
        static int        blocks_per_sm[64] = {};
        static int        sm_count[64]      = {};
        static std::mutex mtx;
        int               dev = 0;
        cudaGetDevice(&dev);
        if(dev < 0 || dev >= 64)
            return cudaErrorInvalidDevice;
        auto kern = stockham_fused2d_kernel<C, UN>;
        {
            std::lock_guard<std::mutex> g(mtx);
            if(!blocks_per_sm[dev])
            {
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F::SMEM_BYTES);
                if(e != cudaSuccess)
                    return e;
                int nb = 0;
                e      = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kern, F::THREADS, F::SMEM_BYTES);
                if(e != cudaSuccess)
                    return e;
                cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
                blocks_per_sm[dev] = nb > 0 ? nb : 1;
            }
        }
        if(nimages == 0)
            return cudaSuccess;
        if(nimages > 0x7ffffffeull || !a.aux[1])
            return cudaErrorInvalidValue;
        tmap_encode_fn enc = tmap_encoder();
        if(!enc)
            return cudaErrorNotSupported;
        // the output array as a tensor: columns, rows (the column transform's dimension), images
        const cuuint64_t ce  = sizeof(T2) / 8;
        const cuuint64_t row = (cuuint64_t)C::N * sizeof(T2);
        cuuint64_t       istr = (cuuint64_t)a.out.os[1] * sizeof(T2);
        if(nimages == 1 || a.out.os[1] <= 0)
            istr = row * C::N;
        if(istr < row)
            return cudaErrorInvalidValue;
        const cuuint64_t dims[4]    = {(cuuint64_t)C::N * ce, (cuuint64_t)C::N, (cuuint64_t)nimages, 1};
        const cuuint64_t strides[3] = {row, istr, istr * nimages};
        const cuuint32_t box[4]     = {(cuuint32_t)(CC::ROW_BYTES / 8), (cuuint32_t)CC::BOX_ROWS, 1, 1};
        const cuuint32_t estr[4]    = {1, 1, 1, 1};
        alignas(64) CUtensorMap map;
        if(enc(&map,
               CU_TENSOR_MAP_DATA_TYPE_UINT64,
               4,
               a.out.p[0],
               dims,
               strides,
               box,
               estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
           != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
        b200fft_kargs ka = a;
        ka.on[1]         = (unsigned)nimages;
        ka.out.es        = C::N; // rows back to back
        ka.iaux[3]       = 0 | (1 << 2) | (2 << 4); // transform = dimension 1, images = dimension 2
        // the per-image counters start at zero
        cudaError_t e = cudaMemsetAsync(const_cast<void*>(a.aux[1]), 0, sizeof(int) * nimages, stream);
        if(e != cudaSuccess)
            return e;
        unsigned long long grid  = (unsigned long long)blocks_per_sm[dev] * sm_count[dev];
        // distance (in images) between the row tiles and the column tiles handed out together; every image in
        // flight lives in L2 meanwhile.  Measured on 1024 x 1024 images: double precision (16 MB per image) is
        // fastest at 1 (0.668 ms per 64 images; 0.675 / 0.716 / 0.741 at 2 / 3 / 4), single precision at 3
        // (1.376 ms per 256 images; 1.486 / 1.424 / 1.403 at 1 / 2 / 4).  B200FFT_2D_L2_DEPTH overrides.
        static const char* depth_env = getenv("B200FFT_2D_L2_DEPTH");
        unsigned long long depth     = sizeof(T2) == 8 ? 3 : 1;
        if(depth_env && atoi(depth_env) >= 1 && atoi(depth_env) <= 16)
            depth = (unsigned long long)atoi(depth_env);
        ka.iaux[2] = (long long)depth;
        const unsigned long long items = (nimages + depth) * (unsigned long long)(F::TR + F::TC);
        if(grid > items)
            grid = items;
        // CTAs wait for one another's row tiles: all of them must be resident, hence a cooperative launch
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim            = dim3((unsigned)grid);
        cfg.blockDim           = dim3(F::THREADS);
        cfg.dynamicSmemBytes   = F::SMEM_BYTES;
        cfg.stream             = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id              = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.attrs               = attr;
        cfg.numAttrs            = 1;
        return cudaLaunchKernelEx(&cfg, kern, ka, map);
    }
} // namespace b200fft
