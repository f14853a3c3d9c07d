/*
 * rocfft_b200_ext.h — entry points of librocfft.so that have no counterpart in
 * the reference's rocfft.h.  They exist for inspection and testing; a program
 * written against rocfft.h alone never needs them.
 */
#ifndef ROCFFT_B200_EXT_H
#define ROCFFT_B200_EXT_H

#include "rocfft/rocfft.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Text description of a plan: one line per kernel launch with the kernel name,
 * the buffers it reads and writes, tile counts and strides.  The same text
 * rocfft_plan_get_print writes to stdout (reference: library/src/plan.cpp:3147,
 * plan log layer at :3757-3914), returned in a caller buffer instead. */
ROCFFT_EXPORT rocfft_status b200fft_plan_describe(const rocfft_plan plan, char* buf, size_t len);

/* Kernels that wait on hardware barriers (the bulk-copy row kernels and the
 * cluster column kernels) bound every wait; when a wait gives up the kernel sets
 * a flag in plan-owned device memory and carries on so that the launch still
 * ends.  This call synchronises with the device (a blocking 4-byte copy per
 * flag) and sets *raised to 1 if any kernel of the plan has ever raised its
 * flag; results of such an execute are not valid.  No reference counterpart:
 * the reference's kernels have no such waits. */
ROCFFT_EXPORT rocfft_status b200fft_plan_device_error(const rocfft_plan plan, int* raised);

/* Host copy of the stacked per-pass twiddle table a Stockham kernel with the
 * given factor list reads (reference layout: library/src/twiddles.cpp:68-106).
 * precision 0 = float pairs, 1 = double pairs.  *needed receives the byte size. */
ROCFFT_EXPORT rocfft_status b200fft_stacked_twiddles(
    int n, const int* factors, int nfactors, int precision, void* out, size_t out_bytes, size_t* needed);

/* Enumerates the function pool (reference: library/src/include/function_pool.h:44-272). */
ROCFFT_EXPORT rocfft_status b200fft_pool_query(
    size_t index, int* length, int* precision, int* variant, int* factors8, size_t* count);

/* NCCL communicator helpers for multi-process plans (one process per GPU).
 * The reference takes an MPI communicator through
 * rocfft_plan_description_set_comm(desc, rocfft_comm_mpi, &comm)
 * (library/src/plan.cpp:356-395); this library takes
 * rocfft_comm_nccl with a pointer to an ncclComm_t.  These three calls let a
 * program that does not link NCCL itself build one: rank 0 creates the
 * 128-byte id, the program ships it to the other ranks by any means, and every
 * rank creates its communicator (collective call). */
ROCFFT_EXPORT rocfft_status b200fft_nccl_unique_id(void* id128);
ROCFFT_EXPORT rocfft_status b200fft_nccl_comm_create(int nranks, int rank, const void* id128, void** comm);
ROCFFT_EXPORT rocfft_status b200fft_nccl_comm_destroy(void* comm);

/* Batched 1D complex transform that allocates no device memory, for callers
 * that may not call cudaMalloc where they run the transform (a real-time
 * loop that must not take the allocator's locks, a process whose device
 * memory was handed out once and frozen, ...).  It has no counterpart in the
 * reference: rocFFT always allocates twiddle tables at plan creation and may
 * allocate a work buffer at execute time.
 *
 * Single precision, interleaved, unit stride, `batch` rows of `length` points
 * back to back; in == out is allowed.  `length` must be a power of two from 256
 * to 524288 and length * batch * 8 bytes must not exceed 4 MiB
 * (rocfft_status_invalid_arg_value otherwise): the intermediate array lives in a
 * 4 MiB + 64 KiB __device__ array inside the library image, which every GPU
 * that loads the library holds until the process exits.  `stream` is a
 * cudaStream_t.  The first call on a device, and the first call after `length`
 * changes, rewrites small tables in that array: it waits for `stream` to drain,
 * copies the tables on `stream` and waits again — make that call before any
 * stream capture begins; calls that keep `length` never synchronise.  All calls
 * share the array: calls that overlap on the GPU (other streams, other host
 * threads) race, so serialise them. */
ROCFFT_EXPORT rocfft_status b200fft_c2c_1d_static_scratch(
    const void* in, void* out, size_t length, size_t batch, int inverse, void* stream);

/* The exchange schedule of a slab-decomposed 3D plan, as pure host arithmetic:
 * byte offsets (relative to the send buffer and to the receive buffer) and the
 * size of the block exchanged with each of `ranks` peers in chunk `chunk` of the
 * first (`first` != 0) or second global transpose.  This is the function the
 * executor itself calls (reference counterpart: the offsets built in
 * GlobalTransposeA2A, library/src/plan.cpp:2033-2220); it is exported so that the
 * decomposition can be tested without GPUs. */
ROCFFT_EXPORT rocfft_status b200fft_slab_exchange_offsets(int     ranks,
                                                          int     chunks,
                                                          size_t  slab_bytes,
                                                          int     first,
                                                          int     chunk,
                                                          size_t* send_off,
                                                          size_t* recv_off,
                                                          size_t* block_bytes);

/* The same for a rank-2 transform on row slabs (rank q holds rows [q*ny/ranks, (q+1)*ny/ranks) of
 * every image): byte offsets at which rank `rank` stores into EVERY peer's receive buffers — in the
 * first phase its rows of the peer's T[y][x_local] (x_local = the peer's nx/ranks columns), in the
 * second its columns of the peer's row buffer [y_local][x].  Called by the plan builder; exported
 * for the same reason (reference counterpart as above). */
ROCFFT_EXPORT rocfft_status b200fft_rows2d_exchange_offsets(
    int ranks, int rank, size_t nx, size_t ny, size_t elem_bytes, size_t* first_off, size_t* second_off);

/* Number of GPU kernels this library has launched in the calling process. */
ROCFFT_EXPORT unsigned long long b200fft_launch_count();

/* Profiling aid in the spirit of the reference's profile log layer
 * (library/src/powX.cpp:817-883): runs the plan once with a CUDA event between
 * consecutive kernel launches, synchronises, and writes each step's device time
 * in milliseconds to step_ms[0 .. *nsteps).  A plan that needs a work buffer
 * must be given one through `info`. */
ROCFFT_EXPORT rocfft_status b200fft_execute_profiled(const rocfft_plan     plan,
                                                     void*                 in_buffer[],
                                                     void*                 out_buffer[],
                                                     rocfft_execution_info info,
                                                     float*                step_ms,
                                                     size_t                max_steps,
                                                     size_t*               nsteps);

#ifdef __cplusplus
}
#endif
#endif
