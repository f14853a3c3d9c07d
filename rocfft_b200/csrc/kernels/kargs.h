// Kernel-argument structures shared by host code (planner / launch layer) and
// device code.  Plain C structs: they cross the C-ABI launch layer by value.
//
// Role in the reference: library/src/kargs.cpp:28-66 packs lengths / input
// strides / output strides into a device array for every leaf kernel.  Here the
// arguments travel in the kernel parameter space instead (no device allocation,
// no copy at plan time).
#ifndef B200FFT_KARGS_H
#define B200FFT_KARGS_H

#ifdef __cplusplus
extern "C" {
#endif

// One side (input or output) of a batched 1D transform stage.
// All strides are in elements of the view's own element type: complex pairs for
// interleaved data, scalars for planar and real data.
typedef struct b200fft_ioview
{
    void*     p[2]; // [0] interleaved/real base or real plane; [1] imaginary plane (planar)
    long long es; // stride between consecutive points of one transform
    long long os[3]; // strides of the three outer (batch-like) dimensions
    int       planar; // 0 interleaved (or real), 1 planar
    // Two-level stride along the transform, honoured on the output side of the
    // "blocked output" kernel variants only: point e lives at
    // (e / blk) * bs + (e % blk) * es.  Used to write a transform dimension that
    // is split into per-rank blocks of a packed exchange buffer.
    unsigned  blk;
    unsigned  blk_mul; // ceil(2^32 / blk), for an exact multiply-high division
    int       pad_;
    long long bs;
    // Optional table with one base pointer per block (blocked-output variants): block q is
    // written at blk_ptrs[q] instead of p[0] + q * bs.  The multi-device layer points the
    // entries at peer GPUs' receive buffers, so the FFT pass stores its result straight
    // into the other ranks' memory over NVLink.
    void* const* blk_ptrs;
} b200fft_ioview;

// Arguments of every Stockham tile kernel.
typedef struct b200fft_kargs
{
    b200fft_ioview in;
    b200fft_ioview out;
    unsigned       on[3]; // outer lengths; on[0] is the dimension tiles run along
    unsigned       ntile0; // ceil(on[0] / transforms-per-block)
    int            inverse; // 0 forward (exp(-i..)), 1 inverse (exp(+i..)), unnormalised
    int            use_scale; // multiply every output by `scale`
    double         scale;
    const void*    twiddles; // stacked per-pass twiddle table in the kernel's precision
    const void*    aux[4]; // kernel-family specific tables (chirp, large twiddles, ...)
    long long      iaux[4]; // kernel-family specific integers
} b200fft_kargs;

// Arguments of the element-wise helper kernels (real pre/post, Bluestein
// multiplies, copies, transposes).
typedef struct b200fft_eargs
{
    b200fft_ioview in;
    b200fft_ioview out;
    unsigned       n; // points per transform handled by the kernel (meaning per kernel)
    unsigned       on[3];
    int            inverse;
    int            use_scale;
    double         scale;
    const void*    aux[4];
    long long      iaux[4];
} b200fft_eargs;

#ifdef __cplusplus
}
#endif
#endif
