// Executor: resolves buffers and enqueues every step of a plan on a stream.
//
// Role in the reference: library/src/powX.cpp:525-957 (TransformPowX: choose
// each kernel's input/output among user buffers and work-buffer segments, apply
// offsets, launch) and library/src/transform.cpp:361-474 (ExecPlan::ExecuteAsync).
// Nothing here synchronises: all work is asynchronous on the caller's stream.
#include "plan.h"
#include <atomic>
#include <cstdint>

namespace b200fft
{
    namespace
    {
        inline char* bump(void* p, long long bytes)
        {
            return static_cast<char*>(p) + bytes;
        }

        bool resolve(const BufRef& b, void* const* in, void* const* out, void* work, void* p[2])
        {
            void* const* src = nullptr;
            switch(b.id)
            {
            case BUF_USER_IN:
                src = in;
                break;
            case BUF_USER_OUT:
                src = out;
                break;
            case BUF_ABS:
                p[0] = reinterpret_cast<void*>(b.byte_off[0]);
                p[1] = nullptr;
                return true;
            case BUF_TEMP:
                if(!work)
                    return false;
                p[0] = bump(work, (long long)b.byte_off[0]);
                p[1] = nullptr;
                return true;
            }
            if(!src || !src[0])
                return false;
            p[0] = bump(src[0], (long long)b.byte_off[0]);
            p[1] = nullptr;
            if(b.planar)
            {
                if(!src[1])
                    return false;
                p[1] = bump(src[1], (long long)b.byte_off[1]);
            }
            return true;
        }

    }

    std::atomic<unsigned long long> g_launch_count{0};

    static rocfft_status run_steps(const PlanCore&          core,
                                   const std::vector<Step>& steps,
                                   void* const*             in,
                                   void* const*             out,
                                   void*                    work,
                                   cudaStream_t             stream,
                                   cudaEvent_t*             step_events,
                                   StepObserver             observer     = nullptr,
                                   void*                    observer_ctx = nullptr)
    {
        size_t step_index = 0;
        for(const Step& s : steps)
        {
            if(step_events)
                cudaEventRecord(step_events[step_index], stream);
            ++step_index;
            void *ip[2], *op[2];
            if(!resolve(s.in, in, out, work, ip) || !resolve(s.out, in, out, work, op))
                return rocfft_status_failure;
            if(!s.alt.empty()
               && ((reinterpret_cast<uintptr_t>(ip[0]) | reinterpret_cast<uintptr_t>(op[0])) & 15u) != 0)
            {
                // misaligned bases: the ordinary passes this step stands for
                rocfft_status st = run_steps(core, s.alt, in, out, work, stream, nullptr);
                if(st != rocfft_status_success)
                    return st;
                if(observer)
                    observer(observer_ctx, step_index - 1, s, op[0], stream);
                continue;
            }

            // host loops over dimensions the kernels do not index themselves
            std::vector<size_t> idx(s.loops.size(), 0);
            for(;;)
            {
                long long ioff = 0, ooff = 0;
                for(size_t k = 0; k < s.loops.size(); ++k)
                {
                    ioff += (long long)idx[k] * s.loops[k].in_stride;
                    ooff += (long long)idx[k] * s.loops[k].out_stride;
                }
                void* ipp[2] = {bump(ip[0], ioff * (long long)s.in_elem_bytes),
                                ip[1] ? bump(ip[1], ioff * (long long)s.in_elem_bytes) : nullptr};
                void* opp[2] = {bump(op[0], ooff * (long long)s.out_elem_bytes),
                                op[1] ? bump(op[1], ooff * (long long)s.out_elem_bytes) : nullptr};
                cudaError_t e;
                if(s.kind == Step::EW)
                {
                    b200fft_eargs a = s.ea;
                    a.in.p[0]       = ipp[0];
                    a.in.p[1]       = ipp[1];
                    a.out.p[0]      = opp[0];
                    a.out.p[1]      = opp[1];
                    e = b200fft_launch_elementwise(s.ew_kind, core.precision, &a, stream);
                }
                else
                {
                    b200fft_kargs a = s.ka;
                    a.in.p[0]       = ipp[0];
                    a.in.p[1]       = ipp[1];
                    a.out.p[0]      = opp[0];
                    a.out.p[1]      = opp[1];
                    const bool misaligned
                        = ((reinterpret_cast<uintptr_t>(ipp[0]) | reinterpret_cast<uintptr_t>(opp[0])) & 15u) != 0;
                    if(s.kern_unaligned && misaligned)
                    {
                        a.ntile0 = s.ntile0_unaligned;
                        if(s.twiddles_unaligned)
                            a.twiddles = s.twiddles_unaligned;
                        e = s.kern_unaligned->launch(&a, s.ntiles_unaligned, stream);
                    }
                    else
                        e = s.kern->launch(&a, s.ntiles, stream);
                }
                if(e != cudaSuccess)
                    return rocfft_status_failure;
                g_launch_count.fetch_add(1, std::memory_order_relaxed);

                size_t k = 0;
                for(; k < idx.size(); ++k)
                {
                    if(++idx[k] < s.loops[k].count)
                        break;
                    idx[k] = 0;
                }
                if(k == idx.size())
                    break;
            }
            if(observer)
                observer(observer_ctx, step_index - 1, s, op[0], stream);
        }
        if(step_events)
            cudaEventRecord(step_events[step_index], stream);
        return rocfft_status_success;
    }

    rocfft_status execute_core(const PlanCore& core,
                               void* const*    in,
                               void* const*    out,
                               void*           work,
                               cudaStream_t    stream,
                               cudaEvent_t*    step_events,
                               StepObserver    observer,
                               void*           observer_ctx)
    {
        if(core.host_only)
            return rocfft_status_failure; // no CPU fallback exists
        return run_steps(core, core.steps, in, out, work, stream, step_events, observer, observer_ctx);
    }
}
