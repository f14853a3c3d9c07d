/* A plain C11 client of librocfft.so: the canonical rocFFT call sequence
 * (description -> layout -> plan -> info -> work buffer -> execute; reference:
 * shared/rocfft_params.h:341-503) on a 4096-point batched complex transform, with device memory from
 * the CUDA runtime.  Compiled against include/rocfft/rocfft.h only — no C++ and no Python — to show
 * that the header is a C header and the library a drop-in for C consumers.
 * Checks the result against a direct evaluation of a few output bins and prints "c_client ok". */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <cuda_runtime_api.h>

#include "rocfft/rocfft.h"

#define N 4096
#define BATCH 8
#define CHECK(call)                                                  \
    do                                                               \
    {                                                                \
        rocfft_status s_ = (call);                                   \
        if(s_ != rocfft_status_success)                              \
        {                                                            \
            fprintf(stderr, "%s -> status %d\n", #call, (int)s_);  \
            return 1;                                                \
        }                                                            \
    } while(0)

int main(void)
{
    const size_t total = (size_t)N * BATCH;
    float*       h     = (float*)malloc(total * 2 * sizeof(float));
    float*       g     = (float*)malloc(total * 2 * sizeof(float));
    unsigned     seed  = 12345u;
    for(size_t i = 0; i < total * 2; ++i)
    {
        seed = seed * 1664525u + 1013904223u;
        h[i] = (float)((seed >> 8) & 0xffff) / 65536.0f - 0.5f;
    }
    void* d_in  = NULL;
    void* d_out = NULL;
    if(cudaMalloc(&d_in, total * 2 * sizeof(float)) != cudaSuccess || cudaMalloc(&d_out, total * 2 * sizeof(float)) != cudaSuccess)
        return 2;
    cudaMemcpy(d_in, h, total * 2 * sizeof(float), cudaMemcpyHostToDevice);

    CHECK(rocfft_setup());
    char version[64];
    CHECK(rocfft_get_version_string(version, sizeof version));

    rocfft_plan_description desc = NULL;
    CHECK(rocfft_plan_description_create(&desc));
    size_t strides[1] = {1};
    size_t offsets[1] = {0};
    CHECK(rocfft_plan_description_set_data_layout(desc,
                                                  rocfft_array_type_complex_interleaved,
                                                  rocfft_array_type_complex_interleaved,
                                                  offsets,
                                                  offsets,
                                                  1,
                                                  strides,
                                                  N,
                                                  1,
                                                  strides,
                                                  N));
    size_t      lengths[1] = {N};
    rocfft_plan plan       = NULL;
    CHECK(rocfft_plan_create(&plan,
                             rocfft_placement_notinplace,
                             rocfft_transform_type_complex_forward,
                             rocfft_precision_single,
                             1,
                             lengths,
                             BATCH,
                             desc));
    CHECK(rocfft_plan_description_destroy(desc)); /* the plan holds its own copy */

    rocfft_execution_info info = NULL;
    CHECK(rocfft_execution_info_create(&info));
    size_t work_bytes = 0;
    CHECK(rocfft_plan_get_work_buffer_size(plan, &work_bytes));
    void* work = NULL;
    if(work_bytes)
    {
        if(cudaMalloc(&work, work_bytes) != cudaSuccess)
            return 2;
        CHECK(rocfft_execution_info_set_work_buffer(info, work, work_bytes));
    }
    cudaStream_t stream;
    cudaStreamCreate(&stream);
    CHECK(rocfft_execution_info_set_stream(info, stream));

    void* in_ptrs[1]  = {d_in};
    void* out_ptrs[1] = {d_out};
    CHECK(rocfft_execute(plan, in_ptrs, out_ptrs, info));
    if(cudaStreamSynchronize(stream) != cudaSuccess)
        return 2;
    cudaMemcpy(g, d_out, total * 2 * sizeof(float), cudaMemcpyDeviceToHost);

    /* direct DFT of a few bins of a few rows, in double precision */
    const int    bins[4] = {0, 1, N / 2, N - 1};
    const double pi      = 3.14159265358979323846;
    double       worst   = 0.0;
    for(int b = 0; b < BATCH; b += 3)
        for(int q = 0; q < 4; ++q)
        {
            double re = 0.0, im = 0.0;
            for(int n = 0; n < N; ++n)
            {
                const double a  = -2.0 * pi * (double)((long long)n * bins[q] % N) / (double)N;
                const double xr = h[2 * ((size_t)b * N + n)], xi = h[2 * ((size_t)b * N + n) + 1];
                re += xr * cos(a) - xi * sin(a);
                im += xr * sin(a) + xi * cos(a);
            }
            const double dr = g[2 * ((size_t)b * N + bins[q])] - re, di = g[2 * ((size_t)b * N + bins[q]) + 1] - im;
            const double e  = sqrt(dr * dr + di * di);
            if(e > worst)
                worst = e;
        }
    /* rocfft-test's Linf bound with |ref|_inf <= N / sqrt(2): eps * |ref|_inf * ln N */
    const double cut = 3.75e-5 * 64.0 * log((double)N);
    CHECK(rocfft_execution_info_destroy(info));
    CHECK(rocfft_plan_destroy(plan));
    CHECK(rocfft_cleanup());
    cudaFree(d_in);
    cudaFree(d_out);
    if(work)
        cudaFree(work);
    if(!(worst <= cut))
    {
        fprintf(stderr, "c_client: worst error %g above %g\n", worst, cut);
        return 3;
    }
    printf("c_client ok (%s, worst error %.3g)\n", version, worst);
    return 0;
}
