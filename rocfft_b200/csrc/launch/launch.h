// Thin C-ABI launch layer between the C++ planner and the CUDA kernels.
//
// Role in the reference: library/src/include/function_pool.h:44-272 (lookup of a
// kernel by length / precision / scheme) and library/src/rtc_kernel.cpp:58-115
// (packing arguments and launching).  The planner is plain C++ and never sees
// a <<< >>> launch: it looks kernels up in the pool and calls the function
// pointers below with plain structs, sizes and a stream.
#ifndef B200FFT_LAUNCH_H
#define B200FFT_LAUNCH_H

#include "../kernels/kargs.h"
#include <cuda_runtime_api.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// Tiling / addressing variants of a Stockham kernel (reference schemes in
// library/src/include/compute_scheme.h:29-83 given for orientation).
typedef enum b200fft_variant
{
    B200FFT_ROW_UNIT = 0, // rows in, rows out, interleaved unit stride  (CS_KERNEL_STOCKHAM)
    B200FFT_ROW_GEN  = 1, // rows, any stride / planar
    B200FFT_COL_STR  = 2, // columns in, columns out, interleaved  (CS_KERNEL_STOCKHAM_BLOCK_CC)
    B200FFT_COL_GEN  = 3, // columns, any stride / planar
    B200FFT_ROW_TOUT = 4, // rows in, columns out (transposing store) (CS_KERNEL_STOCKHAM_BLOCK_RC)
    B200FFT_COL_ROUT = 5, // columns in, rows out                     (CS_KERNEL_STOCKHAM_BLOCK_CR)
    B200FFT_COL_BLK  = 6, // columns, output split into per-rank blocks (multi-device exchange buffers)
    B200FFT_ROW_R2C  = 7, // rows of packed reals in, Hermitian rows out (length = half the real length)
    B200FFT_ROW_C2R  = 8, // Hermitian rows in, rows of packed reals out
    B200FFT_ROW_BLUE = 9, // whole Bluestein transform in one kernel; `length` is the padded length M
    // persistent kernels that move contiguous row tiles with the bulk-copy engine (TMA);
    // they need 16-byte aligned base pointers and back-to-back rows
    B200FFT_ROW_TMA     = 10,
    B200FFT_ROW_R2C_TMA = 11,
    B200FFT_ROW_C2R_TMA = 12,
    // single-precision column tiles with two adjacent columns per thread (128-bit accesses);
    // need even strides, an even column count and 16-byte aligned bases
    B200FFT_COL_PAIR     = 13,
    B200FFT_COL_PAIR_BLK = 14,
    // persistent column kernels with 128-byte-wide tiles loaded by the tensor copy engine
    // (stockham_colstream.cuh); column count must be a multiple of the tile width
    B200FFT_COL_TMA     = 15,
    B200FFT_COL_TMA_BLK = 16,
    // 128-byte-wide column tiles shared by a cluster of two CTAs through distributed shared
    // memory (stockham_colcluster.cuh); power-of-two lengths
    B200FFT_COL_CL     = 17,
    B200FFT_COL_CL_BLK = 18,
    // 19: whole small 2D transforms (B200FFT_2D_SINGLE, separate table below)
    // real transforms of odd length as one full-length complex kernel: real rows in / Hermitian
    // half out, and Hermitian half in (rebuilt by conjugate symmetry) / real rows out
    B200FFT_ROW_R2C_FULL = 20,
    B200FFT_ROW_C2R_FULL = 21,
    // (22: B200FFT_2D_L2, separate table below)
    // persistent TMA row kernels working on pairs of rows in packed single precision
    // (two rows per thread slot, one packed instruction for both); tpb = rows per tile
    B200FFT_ROW_TMA_PK     = 23,
    B200FFT_ROW_R2C_TMA_PK = 24,
    B200FFT_ROW_C2R_TMA_PK = 25,
    // whole Bluestein transform in one kernel, padded length = rows x 1024, one warp per row (bluestein_rc.cuh);
    // `length` is the padded length
    B200FFT_ROW_BLUE_RC = 27,
} b200fft_variant;

typedef cudaError_t (*b200fft_tile_launcher)(const b200fft_kargs*, unsigned long long ntiles, cudaStream_t);

typedef struct b200fft_pool_entry
{
    int                   length;
    int                   precision; // 0 single, 1 double
    int                   variant; // b200fft_variant
    int                   tpt; // threads per transform
    int                   tpb; // transforms per block (tile width)
    int                   threads;
    int                   nfactors;
    int                   factors[8];
    unsigned long long    smem_bytes;
    b200fft_tile_launcher launch;
    const char*           name;
} b200fft_pool_entry;

// generated table of every compiled Stockham kernel
const b200fft_pool_entry* b200fft_pool(size_t* count);

// whole small 2D transforms in one kernel (kernels/stockham_2d.cuh).  `base` describes the row
// phase (length = n0 * n1 points per image, factors of n0); the launcher's tile count is the
// number of images.
#define B200FFT_2D_SINGLE 19
// whole batches of n0 x n1 images in one persistent kernel that keeps the intermediate array in L2
// (kernels/stockham_fused2d.cuh): same table, `base.tpb` = 16-byte units per tile row
#define B200FFT_2D_L2 22
typedef struct b200fft_pool2d_entry
{
    b200fft_pool_entry base;
    int                n0, n1; // n0 = fastest dimension
    int                nfactors1;
    int                factors1[8]; // factors of n1
} b200fft_pool2d_entry;
const b200fft_pool2d_entry* b200fft_pool2d(size_t* count);

// ---- element-wise helper kernels (elementwise.cu) -------------------------
// Every launcher enqueues on `stream` and returns the launch status.
typedef enum b200fft_ew_kind
{
    B200FFT_EW_COPY_C2C = 0, // complex -> complex copy between layouts (optionally scaled)
    B200FFT_EW_R2C_COPY, // real -> complex (imaginary part zero)
    B200FFT_EW_C2R_COPY, // complex -> real (real part only)
    B200FFT_EW_C2HERM_COPY, // first n/2+1 points of a complex row
    B200FFT_EW_HERM2C_COPY, // Hermitian half -> full complex row
    B200FFT_EW_R2C_POST, // even-length real forward post-processing
    B200FFT_EW_C2R_PRE, // even-length real inverse pre-processing
    B200FFT_EW_BLUE_PAD_MUL, // x * chirp, zero padded to M
    B200FFT_EW_POINT_MUL, // row *= table
    B200FFT_EW_BLUE_RES_MUL, // first n points of row * chirp
    B200FFT_EW_LARGE_TWIDDLE, // row-major [n1][n2] tile *= W_n^(i1*i2)
    B200FFT_EW_COUNT
} b200fft_ew_kind;

cudaError_t b200fft_launch_elementwise(int kind, int precision, const b200fft_eargs* a, cudaStream_t stream);

// order-independent 64-bit checksum of `bytes` bytes (8-byte words) into *out (device memory); kernelio log layer
cudaError_t b200fft_launch_hash(const void* p, size_t bytes, unsigned long long* out, cudaStream_t stream);

// strided box copy between a brick and the full field (launch/brick_copy.cu); elem_bytes 4 / 8 / 16,
// four extents and element strides per side, fastest dimension first
cudaError_t b200fft_launch_brick_copy(void*                     dst,
                                      const void*               src,
                                      int                       elem_bytes,
                                      const unsigned long long* n,
                                      const long long*          dst_stride,
                                      const long long*          src_stride,
                                      cudaStream_t              stream);

#ifdef __cplusplus
}
#endif
#endif
