// Probe for the wait-expiry test: the library's own kernel sources built with a short spin limit
// (B200FFT_MBAR_SPIN) and with B200FFT_TEST_EXTRA_TX added to every expected transaction count, so
// that every copy lands but no load phase ever completes.  Each kernel must then give up its
// bounded wait, raise the device error flag and return; nothing hangs and nothing faults.
// Prints one line per kernel: "<name> flag=<0|1> status=<cuda error string>".
#include <cstdio>
#include <vector>
#include "gen_butterflies.cuh"
#include "stockham_colstream.cuh"
#include "plan/plan.h"
using namespace b200fft;

template <class C>
static void* twiddles_for(int precision)
{
    std::vector<char> tw;
    int               f[8];
    for(int i = 0; i < C::NPASS; ++i)
        f[i] = C::FL::get(i);
    host_stacked_twiddles(C::N, f, C::NPASS, precision, tw);
    void* d = nullptr;
    cudaMalloc(&d, tw.size());
    cudaMemcpy(d, tw.data(), tw.size(), cudaMemcpyHostToDevice);
    return d;
}

static void report(const char* name, cudaError_t launch, int* dflag)
{
    cudaError_t sync = cudaDeviceSynchronize();
    int         flag = -1;
    cudaMemcpy(&flag, dflag, sizeof flag, cudaMemcpyDeviceToHost);
    printf("%s flag=%d status=%s\n", name, flag, cudaGetErrorString(launch != cudaSuccess ? launch : sync));
}

int main()
{
    int* dflag = nullptr;
    cudaMalloc(&dflag, sizeof(int));
    {
        // contiguous rows through the bulk-copy pipeline: 64 rows of 256 points
        using C = KCfg<float, 256, 16, 8, false, IO_UNIT, IO_UNIT, COOP_NONE, COOP_NONE, 2, FactorList<16, 16>>;
        const size_t rows = 64;
        float2*      d    = nullptr;
        cudaMalloc(&d, rows * C::N * sizeof(float2));
        cudaMemset(d, 0, rows * C::N * sizeof(float2));
        cudaMemset(dflag, 0, sizeof(int));
        b200fft_kargs a{};
        a.in.p[0] = a.out.p[0] = d;
        a.on[0]                = (unsigned)rows;
        a.on[1] = a.on[2] = 1;
        a.ntile0           = (unsigned)(rows / C::TPB);
        a.twiddles         = twiddles_for<C>(0);
        a.aux[3]           = dflag;
        report("rows_tma", launch_rows_tma_kernel<C, MODE_C2C, 3>(a, a.ntile0, nullptr), dflag);
        cudaFree(d);
    }
    {
        // 256-point columns of a [256][64] array through the tensor-copy column kernel
        using C = KCfg<float, 256, 16, 16, true, IO_STRIDED, IO_STRIDED, COOP_NONE, COOP_NONE, 2, FactorList<16, 16>>;
        const size_t cols = 64;
        float2*      d    = nullptr;
        cudaMalloc(&d, cols * C::N * sizeof(float2));
        cudaMemset(d, 0, cols * C::N * sizeof(float2));
        cudaMemset(dflag, 0, sizeof(int));
        b200fft_kargs a{};
        a.in.p[0] = a.out.p[0] = d;
        a.in.es = a.out.es = (long long)cols;
        a.in.os[0] = a.out.os[0] = 1;
        a.on[0]                  = (unsigned)cols;
        a.on[1] = a.on[2] = 1;
        a.ntile0           = (unsigned)(cols / ColStream<C>::COLS);
        a.twiddles         = twiddles_for<C>(0);
        a.aux[3]           = dflag;
        report("col_tma", launch_colstream_kernel<C, false>(a, a.ntile0, nullptr), dflag);
        cudaFree(d);
    }
    return 0;
}
