// Gather / scatter plans: fields whose bricks all belong to this process.
//
// Role in the reference: the general multi-device plan of library/src/plan.cpp
// (:1244-1580): every input brick is gathered into one contiguous array on a
// single device, an ordinary single-device plan transforms it, and the result is
// scattered to the output bricks.  It accepts any brick layout that tiles the
// field (slabs, pencils, input and output split differently, bricks on one or on
// several devices), any rank and batch, complex and real transforms — the cases
// of clients/tests/multi_device_test.cpp:38-187 — and rejects layouts with
// gaps, overlaps or out-of-range bricks at plan creation
// (multi_device_test.cpp:189-280).
//
// The copies are plain kernels on the plan's device that read / write the bricks
// where they lie; bricks on other devices are reached through peer access
// (enabled at plan creation).  Everything is enqueued on the caller's stream;
// when a brick lives on another device the call waits for the stream before it
// returns, so that work queued on that device afterwards sees the result.
// The optimised slab plan (no gather, FFT passes storing straight into the peers'
// buffers) is the multi-process one in mgpu.cpp.
#include "mgpu.h"
#include "../launch/launch.h"
#include "rocfft_b200_ext.h"
#include <sstream>
#include <stdexcept>

namespace b200fft
{
    namespace
    {
        struct BoxCopy
        {
            unsigned long long n[4];
            long long          full_stride[4], brick_stride[4];
            size_t             full_offset; // elements into the full array
            int                device;
        };

        struct GatherPlan
        {
            MultiDeviceHeader    hdr{1};
            rocfft_plan          inner    = nullptr;
            int                  device   = 0;
            bool                 host_only = false;
            bool                 remote    = false; // some brick lives on another device
            bool                 inplace   = false; // inner plan transforms full_in in place
            void *               full_in = nullptr, *full_out = nullptr;
            size_t               in_bytes = 0, out_bytes = 0;
            int                  in_elem = 8, out_elem = 8; // bytes per element
            std::vector<BoxCopy> gathers, scatters;
        };

        // bricks must tile lattice x batch exactly
        void validate_field(const rocfft_field_t& f, const std::vector<size_t>& len /* rank + 1 entries */)
        {
            if(f.bricks.empty())
                throw std::runtime_error("field has no bricks");
            const size_t dim = len.size();
            long double  vol = 0, want = 1;
            for(size_t l : len)
                want *= (long double)l;
            for(const auto& b : f.bricks)
            {
                if(b.lower.size() != dim || b.upper.size() != dim || b.stride.size() != dim)
                    throw std::runtime_error("brick dimension must be the transform rank + 1 (batch last)");
                long double v = 1;
                for(size_t i = 0; i < dim; ++i)
                {
                    if(b.lower[i] >= b.upper[i] || b.upper[i] > len[i])
                        throw std::runtime_error("brick outside the field");
                    v *= (long double)(b.upper[i] - b.lower[i]);
                }
                vol += v;
            }
            for(size_t a = 0; a < f.bricks.size(); ++a)
                for(size_t b = a + 1; b < f.bricks.size(); ++b)
                {
                    bool overlap = true;
                    for(size_t i = 0; i < dim; ++i)
                        overlap = overlap && f.bricks[a].lower[i] < f.bricks[b].upper[i]
                                  && f.bricks[b].lower[i] < f.bricks[a].upper[i];
                    if(overlap)
                        throw std::runtime_error("bricks overlap");
                }
            if(vol != want)
                throw std::runtime_error("bricks do not cover the field");
        }

        void make_copies(const rocfft_field_t& f, const std::vector<size_t>& len, std::vector<BoxCopy>& out)
        {
            const size_t dim = len.size();
            if(dim > 4)
                throw std::runtime_error("too many dimensions");
            std::vector<size_t> full_stride(dim);
            size_t              s = 1;
            for(size_t i = 0; i < dim; ++i)
            {
                full_stride[i] = s;
                s *= len[i];
            }
            for(const auto& b : f.bricks)
            {
                BoxCopy c{};
                c.full_offset = 0;
                for(size_t i = 0; i < 4; ++i)
                {
                    c.n[i]            = i < dim ? b.upper[i] - b.lower[i] : 1;
                    c.full_stride[i]  = i < dim ? (long long)full_stride[i] : 0;
                    c.brick_stride[i] = i < dim ? (long long)b.stride[i] : 0;
                    if(i < dim)
                        c.full_offset += b.lower[i] * full_stride[i];
                }
                c.device = b.device;
                out.push_back(c);
            }
        }
    }

    void build_gather_scatter_plan(rocfft_plan_t* plan)
    {
        const auto& d = plan->desc;
        const bool  fwd_real = plan->transformType == rocfft_transform_type_real_forward;
        const bool  inv_real = plan->transformType == rocfft_transform_type_real_inverse;
        const bool  real     = fwd_real || inv_real;
        const auto  planar   = [](rocfft_array_type t) {
            return t == rocfft_array_type_complex_planar || t == rocfft_array_type_hermitian_planar;
        };
        if(planar(d.inArrayType) || planar(d.outArrayType))
            throw std::runtime_error("fields need interleaved data");
        if(plan->precision == rocfft_precision_half)
            throw std::runtime_error("half precision is not supported");
        if(plan->userLengths.size() != plan->rank)
            throw std::runtime_error("plan lengths missing");

        // lattices of the two fields in the caller's dimension order, batch last
        std::vector<size_t> in_len = plan->userLengths, out_len = plan->userLengths;
        if(fwd_real)
            out_len[0] = out_len[0] / 2 + 1;
        if(inv_real)
            in_len[0] = in_len[0] / 2 + 1;
        in_len.push_back(plan->batch);
        out_len.push_back(plan->batch);
        validate_field(d.inFields[0], in_len);
        validate_field(d.outFields[0], out_len);
        const bool outer_inplace = plan->placement == rocfft_placement_inplace;
        if(outer_inplace && d.inFields[0].bricks.size() != d.outFields[0].bricks.size())
            throw std::runtime_error("in-place plans need as many output bricks as input bricks");

        auto gp      = std::make_unique<GatherPlan>();
        const int rb = plan->precision == rocfft_precision_single ? 4 : 8;
        gp->in_elem  = fwd_real ? rb : 2 * rb;
        gp->out_elem = inv_real ? rb : 2 * rb;
        make_copies(d.inFields[0], in_len, gp->gathers);
        make_copies(d.outFields[0], out_len, gp->scatters);
        size_t in_count = 1, out_count = 1;
        for(size_t l : in_len)
            in_count *= l;
        for(size_t l : out_len)
            out_count *= l;
        gp->in_bytes  = in_count * gp->in_elem;
        gp->out_bytes = out_count * gp->out_elem;
        gp->inplace   = !real && outer_inplace;

        // the single-device plan on contiguous arrays
        rocfft_plan_description desc = nullptr;
        if(rocfft_plan_description_create(&desc) != rocfft_status_success)
            throw std::runtime_error("description");
        rocfft_status st = rocfft_plan_description_set_data_layout(
            desc, d.inArrayType, d.outArrayType, nullptr, nullptr, 0, nullptr, 0, 0, nullptr, 0);
        if(st == rocfft_status_success && d.scale != 1.0)
            st = rocfft_plan_description_set_scale_factor(desc, d.scale);
        if(st == rocfft_status_success)
            st = rocfft_plan_create(&gp->inner,
                                    gp->inplace ? rocfft_placement_inplace : rocfft_placement_notinplace,
                                    plan->transformType,
                                    plan->precision,
                                    plan->rank,
                                    plan->userLengths.data(),
                                    plan->batch,
                                    desc);
        rocfft_plan_description_destroy(desc);
        if(st != rocfft_status_success)
        {
            if(gp->inner)
                rocfft_plan_destroy(gp->inner);
            throw std::runtime_error("single-device plan for the gathered field could not be created");
        }

        int ndev = 0;
        if(cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
        {
            cudaGetLastError();
            gp->host_only = true; // inspectable only
        }
        else
        {
            cudaGetDevice(&gp->device);
            for(auto* v : {&gp->gathers, &gp->scatters})
                for(const BoxCopy& c : *v)
                {
                    if(c.device < 0 || c.device >= ndev)
                    {
                        rocfft_plan_destroy(gp->inner);
                        throw std::runtime_error("brick on a device that does not exist");
                    }
                    if(c.device == gp->device)
                        continue;
                    gp->remote = true;
                    int ok     = 0;
                    cudaDeviceCanAccessPeer(&ok, gp->device, c.device);
                    if(!ok)
                    {
                        rocfft_plan_destroy(gp->inner);
                        throw std::runtime_error("peer access between the plan's device and a brick's device is required");
                    }
                    const cudaError_t e = cudaDeviceEnablePeerAccess(c.device, 0);
                    if(e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                    {
                        rocfft_plan_destroy(gp->inner);
                        throw std::runtime_error("cudaDeviceEnablePeerAccess failed");
                    }
                    cudaGetLastError();
                }
            if(cudaMalloc(&gp->full_in, gp->in_bytes) != cudaSuccess
               || (!gp->inplace && cudaMalloc(&gp->full_out, gp->out_bytes) != cudaSuccess))
            {
                cudaFree(gp->full_in);
                rocfft_plan_destroy(gp->inner);
                throw std::runtime_error("allocation of the gathered field failed");
            }
            if(gp->inplace)
                gp->full_out = gp->full_in;
        }
        plan->mgpu = gp.release();
    }

    void destroy_gather_scatter_plan(rocfft_plan_t* plan)
    {
        auto* gp = static_cast<GatherPlan*>(plan->mgpu);
        if(!gp)
            return;
        if(gp->full_out && gp->full_out != gp->full_in)
            cudaFree(gp->full_out);
        if(gp->full_in)
            cudaFree(gp->full_in);
        if(gp->inner)
            rocfft_plan_destroy(gp->inner);
        delete gp;
        plan->mgpu = nullptr;
    }

    size_t gather_scatter_work_bytes(const rocfft_plan_t* plan)
    {
        auto*  gp = static_cast<const GatherPlan*>(plan->mgpu);
        size_t w  = 0;
        if(gp && gp->inner)
            rocfft_plan_get_work_buffer_size(gp->inner, &w);
        return w;
    }

    std::string describe_gather_scatter_plan(const rocfft_plan_t* plan)
    {
        auto* gp = static_cast<const GatherPlan*>(plan->mgpu);
        if(!gp)
            return "";
        std::ostringstream o;
        o << "gather/scatter plan: " << gp->gathers.size() << " input bricks -> device " << gp->device << " ("
          << gp->in_bytes << " bytes) -> " << gp->scatters.size() << " output bricks (" << gp->out_bytes << " bytes)"
          << (gp->remote ? ", peer access" : "") << "\n";
        std::vector<char> buf(1 << 16);
        if(b200fft_plan_describe(gp->inner, buf.data(), buf.size()) == rocfft_status_success)
            o << buf.data();
        return o.str();
    }

    void gather_scatter_error_flags(const rocfft_plan_t* plan, std::vector<const int*>& out)
    {
        auto* gp = static_cast<const GatherPlan*>(plan->mgpu);
        if(gp && gp->inner && gp->inner->core && gp->inner->core->dev_error)
            out.push_back(gp->inner->core->dev_error);
    }

    rocfft_status execute_gather_scatter_plan(rocfft_plan_t*                 plan,
                                              void* const*                   in,
                                              void* const*                   out,
                                              const rocfft_execution_info_t* info)
    {
        auto* gp = static_cast<GatherPlan*>(plan->mgpu);
        if(!gp || gp->host_only || !gp->inner)
            return rocfft_status_failure;
        const bool outer_inplace = plan->placement == rocfft_placement_inplace;
        if(!outer_inplace && !out)
            return rocfft_status_failure;
        int cur = 0;
        cudaGetDevice(&cur);
        if(cur != gp->device)
            cudaSetDevice(gp->device);
        cudaStream_t  s  = info->stream;
        rocfft_status st = rocfft_status_success;
        auto          fail = [&](rocfft_status v) {
            if(cur != gp->device)
                cudaSetDevice(cur);
            return v;
        };
        for(size_t i = 0; i < gp->gathers.size(); ++i)
        {
            const BoxCopy& c = gp->gathers[i];
            if(!in[i])
                return fail(rocfft_status_failure);
            char* dst = static_cast<char*>(gp->full_in) + c.full_offset * gp->in_elem;
            if(b200fft_launch_brick_copy(dst, in[i], gp->in_elem, c.n, c.full_stride, c.brick_stride, s) != cudaSuccess)
                return fail(rocfft_status_failure);
            ++g_launch_count;
        }
        {
            rocfft_execution_info_t ei = *info;
            void*                   ib[1] = {gp->full_in};
            void*                   ob[1] = {gp->full_out};
            st = rocfft_execute(gp->inner, ib, gp->inplace ? nullptr : ob, &ei);
            if(st != rocfft_status_success)
                return fail(st);
        }
        void* const* dstp = outer_inplace ? in : out;
        for(size_t j = 0; j < gp->scatters.size(); ++j)
        {
            const BoxCopy& c = gp->scatters[j];
            if(!dstp[j])
                return fail(rocfft_status_failure);
            const char* src = static_cast<const char*>(gp->full_out) + c.full_offset * gp->out_elem;
            if(b200fft_launch_brick_copy(dstp[j], src, gp->out_elem, c.n, c.brick_stride, c.full_stride, s)
               != cudaSuccess)
                return fail(rocfft_status_failure);
            ++g_launch_count;
        }
        if(gp->remote && cudaStreamSynchronize(s) != cudaSuccess)
            return fail(rocfft_status_failure);
        return fail(rocfft_status_success);
    }
}
