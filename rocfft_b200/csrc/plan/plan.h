// Internal plan representation of the B200 FFT library.
//
// Role in the reference: library/src/include/plan.h (rocfft_plan_t,
// rocfft_plan_description_t, bricks and fields) and
// library/src/include/tree_node.h:254-673 (the plan tree).  The reference
// builds a tree of nodes, assigns buffers and fuses kernels afterwards; here
// the planner emits a flat list of steps directly, choosing fused kernels by
// construction, so there is no separate assignment or fusion phase.
#pragma once
#include "../launch/launch.h"
#include "rocfft/rocfft.h"
#include <cstddef>
#include <atomic>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

struct rocfft_brick_t
{
    std::vector<size_t> lower, upper, stride; // dim = rank + 1 entries, batch last
    int                 device = 0;
    int                 rank   = 0; // owning process for multi-process plans
};

struct rocfft_field_t
{
    std::vector<rocfft_brick_t> bricks;
};

struct rocfft_plan_description_t
{
    rocfft_array_type   inArrayType  = rocfft_array_type_unset;
    rocfft_array_type   outArrayType = rocfft_array_type_unset;
    std::vector<size_t> inStrides, outStrides;
    size_t              inDist = 0, outDist = 0;
    size_t              inOffset[2]  = {0, 0};
    size_t              outOffset[2] = {0, 0};
    double              scale        = 1.0;
    rocfft_comm_type    comm_type    = rocfft_comm_none;
    void*               comm_handle  = nullptr;
    std::vector<rocfft_field_t> inFields, outFields;
};

struct rocfft_execution_info_t
{
    void*        workBuffer     = nullptr;
    size_t       workBufferSize = 0;
    cudaStream_t stream         = nullptr;
    void*        load_cb        = nullptr;
    void*        store_cb       = nullptr;
};

namespace b200fft
{
    enum BufId
    {
        BUF_USER_IN  = 0,
        BUF_USER_OUT = 1,
        BUF_TEMP     = 2,
        BUF_ABS      = 3, // a fixed device address owned by the plan (byte_off[0] holds it)
    };

    // where a view's base pointer(s) come from at execute time
    struct BufRef
    {
        BufId  id         = BUF_USER_IN;
        size_t byte_off[2] = {0, 0}; // added to pointer 0 / pointer 1 (planar)
        bool   planar     = false;
    };

    enum ElemKind
    {
        EK_CPLX_IL = 0,
        EK_CPLX_PL = 1,
        EK_REAL    = 2,
    };

    // an N-dimensional batched array inside one buffer
    struct DataView
    {
        BufRef                 buf;
        ElemKind               kind = EK_CPLX_IL;
        std::vector<size_t>    len; // per dimension, fastest first
        std::vector<ptrdiff_t> stride;
        size_t                 batch = 1;
        ptrdiff_t              dist  = 0;
    };

    struct LoopDim
    {
        size_t    count;
        ptrdiff_t in_stride, out_stride; // elements of the respective view's type
    };

    struct Step
    {
        enum Kind
        {
            TILE,
            EW,
            FUSED, // special kernels with their own launchers
        } kind
            = TILE;
        const b200fft_pool_entry* kern    = nullptr;
        // when set, `kern` needs 16-byte aligned base pointers and this one is used otherwise
        const b200fft_pool_entry* kern_unaligned = nullptr;
        unsigned                  ntile0_unaligned = 0;
        unsigned long long        ntiles_unaligned = 0;
        const void*               twiddles_unaligned = nullptr; // its own table (the two kernels may factor the length differently)
        int                       ew_kind = 0;
        int                       fused_id = 0;
        b200fft_kargs             ka{};
        b200fft_eargs             ea{};
        BufRef                    in, out;
        size_t                    in_elem_bytes = 0, out_elem_bytes = 0; // for loop pointer bumps
        unsigned long long        ntiles = 0;
        std::vector<LoopDim>      loops; // host-side loops for dimensions beyond the kernel's three
        std::string               note;
        // when not empty: the ordinary steps this step replaces, run instead of it when a base pointer
        // turns out not to be 16-byte aligned at execute time
        std::vector<Step>         alt;
    };

    // device-resident tables owned by a plan
    struct DeviceTable
    {
        void*  ptr   = nullptr;
        size_t bytes = 0;
    };

    struct PlanCore
    {
        int               precision = 0; // 0 single, 1 double
        std::vector<Step> steps;
        size_t            work_bytes = 0;
        std::vector<void*> tables; // cudaMalloc'd, freed with the plan
        int               device = 0;
        bool              host_only = false; // built without a GPU: inspectable, not executable
        int*              dev_error = nullptr; // raised by kernels whose bounded waits expire
        ~PlanCore();
    };
}

struct rocfft_plan_t
{
    size_t                    rank = 0;
    std::vector<size_t>       lengths, outputLengths;
    std::vector<size_t>       userLengths; // as passed to rocfft_plan_create, before dimensions are sorted
    size_t                    batch = 1;
    rocfft_result_placement   placement = rocfft_placement_inplace;
    rocfft_transform_type     transformType = rocfft_transform_type_complex_forward;
    rocfft_precision          precision = rocfft_precision_single;
    rocfft_plan_description_t desc;
    std::unique_ptr<b200fft::PlanCore> core;
    void*                     mgpu = nullptr; // multi-device plan (mgpu/), owned
};

namespace b200fft
{
    // builds plan->core from the normalised description; throws std::runtime_error
    void build_single_device_plan(rocfft_plan_t* plan);
    // runs every step of `core` on `stream`
    // called after every top-level step has been enqueued, with the step's resolved output pointer (kernelio log layer)
    typedef void (*StepObserver)(void* ctx, size_t index, const Step& step, void* out_ptr, cudaStream_t stream);
    rocfft_status execute_core(const PlanCore& core,
                               void* const*    in,
                               void* const*    out,
                               void*           work,
                               cudaStream_t    stream,
                               cudaEvent_t*    step_events = nullptr, // steps+1 events when profiling
                               StepObserver    observer    = nullptr,
                               void*           observer_ctx = nullptr);
    std::string describe_core(const PlanCore& core);
    extern std::atomic<unsigned long long> g_launch_count; // kernels launched by this library

    // host-side table builders (long double internally)
    // `out` receives interleaved (re, im) pairs in the requested precision
    void host_stacked_twiddles(int n, const int* factors, int nfactors, int precision, std::vector<char>& out);
    void host_half_twiddles(size_t n_real, int precision, std::vector<char>& out); // exp(-2 pi i p/n_real), p <= n_real/4
    void host_large_twiddles(size_t n, int precision, int* steps, std::vector<char>& out); // base-256 stepped table
    void host_chirp(size_t n, int precision, std::vector<char>& out); // exp(-i pi p^2/n), p < n
    void host_bluestein_filter(size_t n, size_t m, int precision, std::vector<char>& out); // FFT_m(wrapped conj chirp)/m
    // the same filter in [k2][k1] order and W_m^(n1 k2) in [k2][n1] order for m = rows x cols (bluestein_rc.cuh)
    void host_bluestein_rc_tables(size_t n, size_t rows, size_t cols, int precision, std::vector<char>& filt, std::vector<char>& twm);
}
