/*
 * rocfft.h — public C interface of the B200-native FFT library.
 *
 * This header declares the same entry points, enumerators and calling
 * conventions as ROCm/rocFFT's library/include/rocfft/rocfft.h so that code
 * written against rocFFT links against this library unchanged.  Device
 * pointers are CUDA device pointers and the stream handed to
 * rocfft_execution_info_set_stream is a cudaStream_t.
 *
 * Each declaration names the reference definition it replaces
 * (file:line inside the rocFFT source tree).
 *
 * Conventions shared by every call:
 *   - lengths[0] is the fastest-varying dimension (column-major lengths);
 *   - strides, distances and offsets count elements of the buffer's own type
 *     (reals for real buffers, complex pairs for interleaved buffers);
 *   - all handles are opaque heap objects made and released by paired calls;
 *   - no exception crosses this boundary: failures are reported as a
 *     rocfft_status value.
 */
#ifndef ROCFFT_H
#define ROCFFT_H

#ifndef ROCFFT_EXPORT
#if defined(__GNUC__)
#define ROCFFT_EXPORT __attribute__((visibility("default")))
#else
#define ROCFFT_EXPORT
#endif
#endif

#ifdef __cplusplus
#include <cstddef>
extern "C" {
#else
#include <stddef.h>
#endif

/* Opaque handles (rocfft.h:45-74 in the reference). */
typedef struct rocfft_plan_t*             rocfft_plan;
typedef struct rocfft_plan_description_t* rocfft_plan_description;
typedef struct rocfft_execution_info_t*   rocfft_execution_info;
typedef struct rocfft_field_t*            rocfft_field;
typedef struct rocfft_brick_t*            rocfft_brick;

/* Status codes; numeric values match the reference (rocfft.h:77-88). */
typedef enum rocfft_status_e
{
    rocfft_status_success,
    rocfft_status_failure,
    rocfft_status_invalid_arg_value,
    rocfft_status_invalid_dimensions,
    rocfft_status_invalid_array_type,
    rocfft_status_invalid_strides,
    rocfft_status_invalid_distance,
    rocfft_status_invalid_offset,
    rocfft_status_invalid_work_buffer,
} rocfft_status;

/* Transform kind (rocfft.h:91-97). */
typedef enum rocfft_transform_type_e
{
    rocfft_transform_type_complex_forward,
    rocfft_transform_type_complex_inverse,
    rocfft_transform_type_real_forward,
    rocfft_transform_type_real_inverse,
} rocfft_transform_type;

/* Arithmetic precision (rocfft.h:100-105).  Half precision is accepted by
 * the type but plans for it are refused by this library. */
typedef enum rocfft_precision_e
{
    rocfft_precision_single,
    rocfft_precision_double,
    rocfft_precision_half,
} rocfft_precision;

/* Result placement (rocfft.h:107-117).  A real-inverse transform may
 * overwrite its input even when the placement is not in-place. */
typedef enum rocfft_result_placement_e
{
    rocfft_placement_inplace,
    rocfft_placement_notinplace,
} rocfft_result_placement;

/* Array formats (rocfft.h:120-128). */
typedef enum rocfft_array_type_e
{
    rocfft_array_type_complex_interleaved,
    rocfft_array_type_complex_planar,
    rocfft_array_type_real,
    rocfft_array_type_hermitian_interleaved,
    rocfft_array_type_hermitian_planar,
    rocfft_array_type_unset,
} rocfft_array_type;

/* Communicator kinds for multi-process plans (rocfft.h:131-135).  The
 * reference knows rocfft_comm_mpi only; this library exchanges data with
 * NCCL, so a third kind takes a pointer to an ncclComm_t. */
typedef enum rocfft_comm_type_e
{
    rocfft_comm_none,
    rocfft_comm_mpi,
    rocfft_comm_nccl,
} rocfft_comm_type;

/* Library set-up / tear-down.  Replaces library/src/auxiliary.cpp:83,140. */
ROCFFT_EXPORT rocfft_status rocfft_setup();
ROCFFT_EXPORT rocfft_status rocfft_cleanup();

/* Create a plan.  Replaces library/src/plan.cpp:3083 (rocfft_plan_create)
 * and :2959 (rocfft_plan_create_internal).  `lengths` holds `dimensions`
 * entries (1..3), fastest first; real transforms always give real lengths.
 * `description` may be NULL. */
ROCFFT_EXPORT rocfft_status rocfft_plan_create(rocfft_plan*                  plan,
                                               rocfft_result_placement       placement,
                                               rocfft_transform_type         transform_type,
                                               rocfft_precision              precision,
                                               size_t                        dimensions,
                                               const size_t*                 lengths,
                                               size_t                        number_of_transforms,
                                               const rocfft_plan_description description);

/* Enqueue a transform on the stream of `info` (or the null stream) and
 * return without synchronising.  Replaces library/src/transform.cpp:331.
 * in_buffer/out_buffer are arrays of device pointers: one for interleaved or
 * real data, two (real part, imaginary part) for planar data, one per local
 * brick when fields are used.  out_buffer is ignored for in-place plans;
 * `info` may be NULL. */
ROCFFT_EXPORT rocfft_status rocfft_execute(const rocfft_plan     plan,
                                           void*                 in_buffer[],
                                           void*                 out_buffer[],
                                           rocfft_execution_info info);

/* Replaces library/src/plan.cpp:3130. */
ROCFFT_EXPORT rocfft_status rocfft_plan_destroy(rocfft_plan plan);

/* Every output element is multiplied by `scale_factor`; non-finite values
 * are refused.  Replaces library/src/plan.cpp:69-77. */
ROCFFT_EXPORT rocfft_status rocfft_plan_description_set_scale_factor(
    rocfft_plan_description description, const double scale_factor);

/* Record array types, offsets, strides and distances.  NULL stride arrays
 * and zero distances select the defaults.  Replaces
 * library/src/plan.cpp:397-470. */
ROCFFT_EXPORT rocfft_status
    rocfft_plan_description_set_data_layout(rocfft_plan_description description,
                                            const rocfft_array_type in_array_type,
                                            const rocfft_array_type out_array_type,
                                            const size_t*           in_offsets,
                                            const size_t*           out_offsets,
                                            const size_t            in_strides_size,
                                            const size_t*           in_strides,
                                            const size_t            in_distance,
                                            const size_t            out_strides_size,
                                            const size_t*           out_strides,
                                            const size_t            out_distance);

/* Fields and bricks (multi-device data decomposition).  Replace
 * library/src/plan.cpp:490-696.  A brick is a box [lower, upper) in the
 * (dims..., batch) index space, column-major, with its own strides, living
 * on device `deviceID`. */
ROCFFT_EXPORT rocfft_status rocfft_field_create(rocfft_field* field);
ROCFFT_EXPORT rocfft_status rocfft_field_destroy(rocfft_field field);

/* Replaces library/src/plan.cpp:3279. */
ROCFFT_EXPORT rocfft_status rocfft_get_version_string(char* buf, size_t len);

/* Replaces library/src/plan.cpp:356-395.  With rocfft_comm_nccl the handle
 * points at an ncclComm_t that spans the ranks owning the bricks. */
ROCFFT_EXPORT rocfft_status rocfft_plan_description_set_comm(rocfft_plan_description description,
                                                             rocfft_comm_type        comm_type,
                                                             void*                   comm_handle);

ROCFFT_EXPORT rocfft_status rocfft_brick_create(rocfft_brick* brick,
                                                const size_t* field_lower,
                                                const size_t* field_upper,
                                                const size_t* brick_stride,
                                                size_t        dim,
                                                int           deviceID);
ROCFFT_EXPORT rocfft_status rocfft_brick_destroy(rocfft_brick brick);
ROCFFT_EXPORT rocfft_status rocfft_field_add_brick(rocfft_field field, rocfft_brick brick);
ROCFFT_EXPORT rocfft_status rocfft_plan_description_add_infield(rocfft_plan_description description,
                                                                rocfft_field            field);
ROCFFT_EXPORT rocfft_status
    rocfft_plan_description_add_outfield(rocfft_plan_description description, rocfft_field field);

/* Bytes of scratch memory a plan needs at execute time.  Replaces
 * library/src/plan.cpp:3137. */
ROCFFT_EXPORT rocfft_status rocfft_plan_get_work_buffer_size(const rocfft_plan plan,
                                                             size_t*           size_in_bytes);

/* Print the plan (steps, kernels, buffers) to stdout.  Replaces
 * library/src/plan.cpp:3147. */
ROCFFT_EXPORT rocfft_status rocfft_plan_get_print(const rocfft_plan plan);

/* Replace library/src/plan.cpp:472-488. */
ROCFFT_EXPORT rocfft_status rocfft_plan_description_create(rocfft_plan_description* description);
ROCFFT_EXPORT rocfft_status rocfft_plan_description_destroy(rocfft_plan_description description);

/* Execution info.  Replace library/src/transform.cpp:35-103.  The info
 * object is read at execute time and not retained. */
ROCFFT_EXPORT rocfft_status rocfft_execution_info_create(rocfft_execution_info* info);
ROCFFT_EXPORT rocfft_status rocfft_execution_info_destroy(rocfft_execution_info info);
ROCFFT_EXPORT rocfft_status rocfft_execution_info_set_work_buffer(rocfft_execution_info info,
                                                                  void*                 work_buffer,
                                                                  const size_t size_in_bytes);
/* `stream` is the cudaStream_t value itself, not its address. */
ROCFFT_EXPORT rocfft_status rocfft_execution_info_set_stream(rocfft_execution_info info,
                                                             void*                 stream);
/* User load/store callbacks are an experimental feature of the reference;
 * the setters exist and validate their arguments, but a plan executed with
 * a callback set reports rocfft_status_failure. */
ROCFFT_EXPORT rocfft_status rocfft_execution_info_set_load_callback(rocfft_execution_info info,
                                                                    void** cb_functions,
                                                                    void** cb_data,
                                                                    size_t shared_mem_bytes);
ROCFFT_EXPORT rocfft_status rocfft_execution_info_set_store_callback(rocfft_execution_info info,
                                                                     void** cb_functions,
                                                                     void** cb_data,
                                                                     size_t shared_mem_bytes);

/* Kernel-cache serialisation.  Replace library/src/rtc_exports.cpp:23-51.
 * Kernels here are compiled ahead of time, so the cache is always empty:
 * serialize yields a zero-length buffer and deserialize accepts anything. */
ROCFFT_EXPORT rocfft_status rocfft_cache_serialize(void** buffer, size_t* buffer_len_bytes);
ROCFFT_EXPORT rocfft_status rocfft_cache_buffer_free(void* buffer);
ROCFFT_EXPORT rocfft_status rocfft_cache_deserialize(const void* buffer, size_t buffer_len_bytes);

#ifdef __cplusplus
}
#endif

#endif /* ROCFFT_H */
