// Strided box copy between a brick and the full field.
//
// Role in the reference: the gather / scatter operations of multi-device plans
// (library/src/plan.cpp:1244-1580, "GatherNode" / "ScatterNode" and their pack
// kernels in library/src/tree_node.cpp:473-700): when a field's brick layout has
// no optimised plan, every brick is copied into one contiguous array on a single
// device, transformed there and copied back out.
//
// One thread moves one element of 4, 8 or 16 bytes; the innermost box dimension
// is the fastest thread index so that accesses coalesce whenever a side has unit
// stride there.  Either pointer may be memory of another GPU of the same process
// (plain peer loads / stores).
#include "launch.h"
#include <stdint.h>

namespace
{
    struct BoxArgs
    {
        unsigned long long n[4]; // box extents, fastest first
        long long          ds[4], ss[4]; // element strides of destination and source
        unsigned long long total;
    };

    template <typename E>
    __global__ void __launch_bounds__(256) brick_copy_kernel(E* __restrict__ dst, const E* __restrict__ src, const BoxArgs a)
    {
        for(unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < a.total; i += gridDim.x * 256ull)
        {
            unsigned long long r  = i;
            const unsigned long long i0 = r % a.n[0];
            r /= a.n[0];
            const unsigned long long i1 = r % a.n[1];
            r /= a.n[1];
            const unsigned long long i2 = r % a.n[2];
            const unsigned long long i3 = r / a.n[2];
            const long long d = (long long)i0 * a.ds[0] + (long long)i1 * a.ds[1] + (long long)i2 * a.ds[2]
                                + (long long)i3 * a.ds[3];
            const long long s = (long long)i0 * a.ss[0] + (long long)i1 * a.ss[1] + (long long)i2 * a.ss[2]
                                + (long long)i3 * a.ss[3];
            dst[d] = src[s];
        }
    }
}

// elem_bytes: 4, 8 or 16.  n / dst_stride / src_stride: 4 entries, fastest dimension first
// (unused dimensions: extent 1).  Strides in elements.
extern "C" cudaError_t b200fft_launch_brick_copy(void*                     dst,
                                                 const void*               src,
                                                 int                       elem_bytes,
                                                 const unsigned long long* n,
                                                 const long long*          dst_stride,
                                                 const long long*          src_stride,
                                                 cudaStream_t              stream)
{
    BoxArgs a;
    a.total = 1;
    for(int d = 0; d < 4; ++d)
    {
        a.n[d]  = n[d];
        a.ds[d] = dst_stride[d];
        a.ss[d] = src_stride[d];
        a.total *= n[d];
    }
    if(a.total == 0)
        return cudaSuccess;
    const unsigned long long want = (a.total + 255) / 256;
    const unsigned           grid = (unsigned)(want < 148ull * 32 ? want : 148ull * 32);
    switch(elem_bytes)
    {
    case 4:
        brick_copy_kernel<float><<<grid, 256, 0, stream>>>((float*)dst, (const float*)src, a);
        break;
    case 8:
        brick_copy_kernel<float2><<<grid, 256, 0, stream>>>((float2*)dst, (const float2*)src, a);
        break;
    case 16:
        brick_copy_kernel<double2><<<grid, 256, 0, stream>>>((double2*)dst, (const double2*)src, a);
        break;
    default:
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}
