// b200fft_c2c_1d_static_scratch: a batched 1D complex transform that performs
// no device allocation at all.
//
// Who needs it: code that runs where cudaMalloc is off limits — inside a
// real-time loop or an interrupt-style callback that must not take the
// allocator's locks, in a process whose memory was handed out once by a
// pool and frozen, or while other work has the device in a state where a
// synchronising allocation would stall it.  The regular path
// (rocfft_plan_create + rocfft_execute) allocates twiddle tables when the plan
// is made and may allocate a work buffer at execute time; this entry point
// does neither.
//
// How: it is the two-kernel N = N1 * N2 decomposition the planner uses for long
// transforms (column FFTs of length N1 into a scratch array, twiddle multiply,
// row FFTs of length N2 written transposed), with the scratch array and every
// table living in one file-scope __device__ array that is part of the library
// image.  Every GPU that loads the library therefore holds
// B200FFT_STATIC_SCRATCH_BYTES + 64 KiB of device memory until the process
// exits.
//
// Limits and rules (also stated in the header):
//   - single precision, interleaved complex, unit stride, rows back to back;
//   - length = N1 * N2 with both factors powers of two between 16 and 1024,
//     and length * batch * 8 bytes <= B200FFT_STATIC_SCRATCH_BYTES (4 MiB):
//     lengths 256 ... 524288 (the longest row that fits the array); anything
//     else is refused with rocfft_status_invalid_arg_value;
//   - the first call on a device, and the first call after the length
//     changes, rewrites the small tables: it waits for `stream` to drain (work
//     queued there earlier may still read the old tables), copies the new tables
//     on `stream` and waits again.  Make that call before starting any stream
//     capture.  Calls that keep the length do not synchronise;
//   - all calls share the one scratch array, which keeps the previous call's
//     contents (nothing in it needs to start at zero: every call overwrites
//     what it reads).  Calls that overlap on the GPU (different streams, or
//     different host threads) race on it: serialise them.
#include "../plan/plan.h"
#include "rocfft_b200_ext.h"
#include <mutex>

#define B200FFT_STATIC_SCRATCH_BYTES (4u << 20)
#define B200FFT_STATIC_TABLE_BYTES (64u << 10)

// scratch for the intermediate array, followed by the tables
static __device__ __align__(256) unsigned char g_static_scratch[B200FFT_STATIC_SCRATCH_BYTES + B200FFT_STATIC_TABLE_BYTES];

namespace
{
    struct DeviceState
    {
        bool   ready       = false;
        char*  base        = nullptr; // device address of g_static_scratch on this device
        size_t table_len   = 0; // transform length the tables currently describe
        size_t off_tw1 = 0, off_tw2 = 0, off_large = 0;
        int    large_steps = 1;
        const b200fft_pool_entry *k1 = nullptr, *k2 = nullptr;
        size_t n1 = 0, n2 = 0;
    };
    DeviceState g_state[64];
    std::mutex  g_mutex;

    const b200fft_pool_entry* find_kernel(size_t n, int variant)
    {
        size_t                    cnt = 0;
        const b200fft_pool_entry* p   = b200fft_pool(&cnt);
        for(size_t i = 0; i < cnt; ++i)
            if((size_t)p[i].length == n && p[i].precision == 0 && p[i].variant == variant)
                return &p[i];
        return nullptr;
    }
}

extern "C" ROCFFT_EXPORT rocfft_status b200fft_c2c_1d_static_scratch(
    const void* in, void* out, size_t length, size_t batch, int inverse, void* stream)
{
    if(!in || !out || length == 0 || batch == 0)
        return rocfft_status_invalid_arg_value;
    if(length > (B200FFT_STATIC_SCRATCH_BYTES / 8) || batch > (B200FFT_STATIC_SCRATCH_BYTES / 8) / length)
        return rocfft_status_invalid_arg_value; // beyond the static scratch array
    if(length & (length - 1))
        return rocfft_status_invalid_arg_value;
    // balanced power-of-two split, both factors in [16, 1024]
    size_t n1 = 1;
    while(n1 * n1 < length)
        n1 <<= 1;
    size_t n2 = length / n1;
    if(n1 > n2)
        std::swap(n1, n2);
    if(n1 < 16 || n2 > 1024)
        return rocfft_status_invalid_arg_value;

    int dev = 0;
    if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return rocfft_status_failure;
    cudaStream_t                s = static_cast<cudaStream_t>(stream);
    std::lock_guard<std::mutex> guard(g_mutex);
    DeviceState&                st = g_state[dev];

    if(!st.ready)
    {
        // In host code the array's name is only a handle: ask the runtime for its
        // address on the current device and hand that to the kernels.
        void* p = nullptr;
        if(cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p)
            return rocfft_status_failure;
        st.base  = static_cast<char*>(p);
        st.ready = true;
    }
    if(st.table_len != length)
    {
        // everything is prepared in locals and committed to the per-device state only after the
        // last step succeeded, so that a failure leaves the previous length fully usable
        const b200fft_pool_entry* k1 = find_kernel(n1, B200FFT_COL_STR);
        const b200fft_pool_entry* k2 = find_kernel(n2, B200FFT_ROW_TOUT);
        if(!k1 || !k2)
            return rocfft_status_failure;
        std::vector<char> t1, t2, tl;
        int               large_steps = 1;
        b200fft::host_stacked_twiddles((int)n1, k1->factors, k1->nfactors, 0, t1);
        b200fft::host_stacked_twiddles((int)n2, k2->factors, k2->nfactors, 0, t2);
        b200fft::host_large_twiddles(length, 0, &large_steps, tl);
        auto         up        = [](size_t v) { return (v + 255) & ~size_t(255); };
        const size_t off_tw1   = B200FFT_STATIC_SCRATCH_BYTES;
        const size_t off_tw2   = off_tw1 + up(t1.size());
        const size_t off_large = off_tw2 + up(t2.size());
        if(off_large + tl.size() > B200FFT_STATIC_SCRATCH_BYTES + B200FFT_STATIC_TABLE_BYTES)
            return rocfft_status_failure;
        // Kernels of an earlier call queued on this stream may still read the old tables, and a
        // blocking copy on the legacy stream would not be ordered against a non-blocking stream:
        // drain the caller's stream, copy on it, and drain again (the host vectors go out of scope).
        // No allocation is involved: the destination is the static array.
        if(cudaStreamSynchronize(s) != cudaSuccess)
            return rocfft_status_failure;
        st.table_len = 0; // the table region is about to change: not valid for any length until committed
        if(cudaMemcpyAsync(st.base + off_tw1, t1.data(), t1.size(), cudaMemcpyHostToDevice, s) != cudaSuccess
           || cudaMemcpyAsync(st.base + off_tw2, t2.data(), t2.size(), cudaMemcpyHostToDevice, s) != cudaSuccess
           || cudaMemcpyAsync(st.base + off_large, tl.data(), tl.size(), cudaMemcpyHostToDevice, s) != cudaSuccess
           || cudaStreamSynchronize(s) != cudaSuccess)
            return rocfft_status_failure;
        st.k1          = k1;
        st.k2          = k2;
        st.off_tw1     = off_tw1;
        st.off_tw2     = off_tw2;
        st.off_large   = off_large;
        st.large_steps = large_steps;
        st.n1          = n1;
        st.n2          = n2;
        st.table_len   = length;
    }

    char* T = st.base; // intermediate array [batch][k1][i2]

    // step 1: column FFTs of length n1 (stride n2), tiles across i2; in -> T
    {
        b200fft_kargs a{};
        a.in.p[0]   = const_cast<void*>(in);
        a.out.p[0]  = T;
        a.in.es     = (long long)n2;
        a.out.es    = (long long)n2;
        a.on[0]     = (unsigned)n2;
        a.on[1]     = (unsigned)batch;
        a.on[2]     = 1;
        a.in.os[0]  = 1;
        a.out.os[0] = 1;
        a.in.os[1]  = (long long)length;
        a.out.os[1] = (long long)length;
        a.ntile0    = (a.on[0] + st.k1->tpb - 1) / st.k1->tpb;
        a.inverse   = inverse ? 1 : 0;
        a.twiddles  = st.base + st.off_tw1;
        if(st.k1->launch(&a, (unsigned long long)a.ntile0 * a.on[1], s) != cudaSuccess)
            return rocfft_status_failure;
    }
    // step 2: multiply element (k1, i2) by exp(-+2 pi i k1 i2 / length), in place on T
    {
        b200fft_eargs e{};
        e.in.p[0]  = T;
        e.out.p[0] = T;
        e.in.es = e.out.es = 1;
        e.n                = (unsigned)length;
        e.on[0]            = (unsigned)batch;
        e.on[1] = e.on[2] = 1;
        e.in.os[0] = e.out.os[0] = (long long)length;
        e.inverse                = inverse ? 1 : 0;
        e.aux[0]                 = st.base + st.off_large;
        e.iaux[0]                = (long long)n2;
        e.iaux[1]                = st.large_steps;
        if(b200fft_launch_elementwise(B200FFT_EW_LARGE_TWIDDLE, 0, &e, s) != cudaSuccess)
            return rocfft_status_failure;
    }
    // step 3: row FFTs of length n2, result k2 of row k1 stored at k1 + n1 * k2; T -> out
    {
        b200fft_kargs a{};
        a.in.p[0]   = T;
        a.out.p[0]  = out;
        a.in.es     = 1;
        a.out.es    = (long long)n1;
        a.on[0]     = (unsigned)n1;
        a.on[1]     = (unsigned)batch;
        a.on[2]     = 1;
        a.in.os[0]  = (long long)n2;
        a.out.os[0] = 1;
        a.in.os[1]  = (long long)length;
        a.out.os[1] = (long long)length;
        a.ntile0    = (a.on[0] + st.k2->tpb - 1) / st.k2->tpb;
        a.inverse   = inverse ? 1 : 0;
        a.twiddles  = st.base + st.off_tw2;
        if(st.k2->launch(&a, (unsigned long long)a.ntile0 * a.on[1], s) != cudaSuccess)
            return rocfft_status_failure;
    }
    return rocfft_status_success;
}
