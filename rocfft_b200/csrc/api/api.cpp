// The exported C API: handle management, argument validation, normalisation of
// the plan description, and dispatch into the planner and executor.
//
// Role in the reference: library/src/plan.cpp:69-696, 2959-3289 (descriptions,
// fields, bricks, plan creation), library/src/transform.cpp:35-103, 331-359
// (execution info, rocfft_execute), library/src/auxiliary.cpp:83-205
// (setup/cleanup and log plumbing), library/src/rtc_exports.cpp:23-51 (cache).
// No exception leaves this file: everything is mapped to a rocfft_status.
#include "../plan/plan.h"
#include "../mgpu/mgpu.h"
#include "rocfft_b200_ext.h"
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <mutex>
#include <sstream>

#define B200FFT_VERSION_STRING "1.0.32.b200"

namespace
{
    // ---- logging (ROCFFT_LAYER bitmask: 1 trace, 2 bench, 4 profile, 8 plan, 16 kernelio, 128 graph;
    // include/logging.h:139-150, auxiliary.cpp:83-137 in the reference) ----
    struct Log
    {
        int           layer = 0;
        std::ofstream trace_file, plan_file, bench_file, profile_file, kernelio_file, graph_file;
        std::ostream& kernelio()
        {
            return kernelio_file.is_open() ? (std::ostream&)kernelio_file : std::cerr;
        }
        std::ostream& graph()
        {
            return graph_file.is_open() ? (std::ostream&)graph_file : std::cerr;
        }
        std::mutex    mtx;
        std::ostream& trace()
        {
            return trace_file.is_open() ? (std::ostream&)trace_file : std::cerr;
        }
        std::ostream& plan()
        {
            return plan_file.is_open() ? (std::ostream&)plan_file : std::cerr;
        }
        std::ostream& bench()
        {
            return bench_file.is_open() ? (std::ostream&)bench_file : std::cerr;
        }
        std::ostream& profile()
        {
            return profile_file.is_open() ? (std::ostream&)profile_file : std::cerr;
        }
        void init()
        {
            std::lock_guard<std::mutex> g(mtx);
            const char*                 l = getenv("ROCFFT_LAYER");
            layer                         = l ? atoi(l) : 0;
            if(const char* p = getenv("ROCFFT_LOG_TRACE_PATH"))
                if(!trace_file.is_open())
                    trace_file.open(p, std::ios::app);
            if(const char* p = getenv("ROCFFT_LOG_PLAN_PATH"))
                if(!plan_file.is_open())
                    plan_file.open(p, std::ios::app);
            if(const char* p = getenv("ROCFFT_LOG_BENCH_PATH"))
                if(!bench_file.is_open())
                    bench_file.open(p, std::ios::app);
            if(const char* p = getenv("ROCFFT_LOG_PROFILE_PATH"))
                if(!profile_file.is_open())
                    profile_file.open(p, std::ios::app);
            if(const char* p = getenv("ROCFFT_LOG_KERNELIO_PATH"))
                if(!kernelio_file.is_open())
                    kernelio_file.open(p, std::ios::app);
            if(const char* p = getenv("ROCFFT_LOG_GRAPH_PATH"))
                if(!graph_file.is_open())
                    graph_file.open(p, std::ios::app);
        }
    };
    Log& log()
    {
        static Log l;
        return l;
    }

    template <typename... A>
    void log_trace(const char* fn, A&&... a)
    {
        Log& l = log();
        if(!(l.layer & 1))
            return;
        std::lock_guard<std::mutex> g(l.mtx);
        std::ostringstream          s;
        s << fn;
        ((s << "," << a), ...);
        l.trace() << s.str() << std::endl;
    }

    // the rocfft-bench command line that reproduces a plan (bench log layer; the reference builds
    // the same line in plan.cpp:698-726): row-major lengths and strides, enumerators as integers
    std::string bench_command(const rocfft_plan_t& p)
    {
        std::ostringstream b;
        b << "rocfft-bench --length ";
        for(auto it = p.userLengths.rbegin(); it != p.userLengths.rend(); ++it)
            b << *it << " ";
        b << "-b " << p.batch << " ";
        if(p.placement == rocfft_placement_notinplace)
            b << "-o ";
        b << "-t " << (int)p.transformType << " --precision "
          << (p.precision == rocfft_precision_single ? "single" : p.precision == rocfft_precision_double ? "double" : "half")
          << " --itype " << (int)p.desc.inArrayType << " --otype " << (int)p.desc.outArrayType << " --istride ";
        for(auto it = p.desc.inStrides.rbegin(); it != p.desc.inStrides.rend(); ++it)
            b << *it << " ";
        b << "--ostride ";
        for(auto it = p.desc.outStrides.rbegin(); it != p.desc.outStrides.rend(); ++it)
            b << *it << " ";
        b << "--idist " << p.desc.inDist << " --odist " << p.desc.outDist << " --ioffset ";
        for(size_t v : p.desc.inOffset)
            b << v << " ";
        b << "--ooffset ";
        for(size_t v : p.desc.outOffset)
            b << v << " ";
        return b.str();
    }

    // peak memory bandwidth for the profile layer: ROCFFT_DEVICE_BW (GB/s) or memory clock x bus width
    // (powX.cpp:218-255 in the reference)
    double max_memory_bandwidth_gbs()
    {
        if(const char* e = getenv("ROCFFT_DEVICE_BW"))
            return atof(e);
        int dev = 0, khz = 0, bits = 0;
        if(cudaGetDevice(&dev) != cudaSuccess
           || cudaDeviceGetAttribute(&khz, cudaDevAttrMemoryClockRate, dev) != cudaSuccess
           || cudaDeviceGetAttribute(&bits, cudaDevAttrGlobalMemoryBusWidth, dev) != cudaSuccess)
            return 0.0;
        return 2.0 * khz * 1e3 * (bits / 8.0) / 1e9;
    }

    size_t offset_count(rocfft_array_type t)
    {
        return (t == rocfft_array_type_complex_planar || t == rocfft_array_type_hermitian_planar) ? 2 : 1;
    }

    // defaults for everything the caller left unset (plan.cpp:87-197 in the reference)
    void init_defaults(rocfft_plan_description_t& d,
                       rocfft_transform_type      tt,
                       rocfft_result_placement    placement,
                       const std::vector<size_t>& len,
                       const std::vector<size_t>& olen)
    {
        const size_t rank = len.size();
        const bool   ip   = placement == rocfft_placement_inplace;
        if(d.inArrayType == rocfft_array_type_unset)
            d.inArrayType = tt == rocfft_transform_type_real_forward   ? rocfft_array_type_real
                            : tt == rocfft_transform_type_real_inverse ? rocfft_array_type_hermitian_interleaved
                                                                       : rocfft_array_type_complex_interleaved;
        if(d.outArrayType == rocfft_array_type_unset)
            d.outArrayType = tt == rocfft_transform_type_real_forward   ? rocfft_array_type_hermitian_interleaved
                             : tt == rocfft_transform_type_real_inverse ? rocfft_array_type_real
                                                                        : rocfft_array_type_complex_interleaved;
        if(d.inStrides.empty())
        {
            d.inStrides.push_back(1);
            if(tt == rocfft_transform_type_real_forward && ip)
            {
                // in-place real forward: rows are padded to hold the Hermitian result
                size_t dist = 2 * olen[0];
                for(size_t i = 1; i < rank; ++i)
                {
                    d.inStrides.push_back(dist);
                    dist *= len[i];
                }
            }
            else
                for(size_t i = 1; i < rank; ++i)
                    d.inStrides.push_back(len[i - 1] * d.inStrides[i - 1]);
        }
        if(d.outStrides.empty())
        {
            d.outStrides.push_back(1);
            if(tt == rocfft_transform_type_real_inverse && ip)
            {
                size_t dist = 2 * len[0];
                for(size_t i = 1; i < rank; ++i)
                {
                    d.outStrides.push_back(dist);
                    dist *= len[i];
                }
            }
            else
                for(size_t i = 1; i < rank; ++i)
                    d.outStrides.push_back(olen[i - 1] * d.outStrides[i - 1]);
        }
        if(d.inDist == 0)
        {
            if(tt == rocfft_transform_type_real_forward && rank == 1 && ip)
                d.inDist = 2 * (len[0] / 2 + 1) * d.inStrides[0];
            else
                d.inDist = len[rank - 1] * d.inStrides[rank - 1];
        }
        if(d.outDist == 0)
        {
            if(tt == rocfft_transform_type_real_inverse && rank == 1 && ip)
                d.outDist = 2 * len[0] * d.outStrides[0];
            else
                d.outDist = olen[rank - 1] * d.outStrides[rank - 1];
        }
    }

    // order dimensions fastest-first by stride and drop trailing unit lengths
    // (plan.cpp:224-285 in the reference); real transforms keep dimension 0
    void sort_dims(rocfft_plan_t& p)
    {
        struct IoDim
        {
            size_t len, olen, is, os;
        };
        const bool c2c = p.transformType == rocfft_transform_type_complex_forward
                         || p.transformType == rocfft_transform_type_complex_inverse;
        const size_t       start = c2c ? 0 : 1;
        std::vector<IoDim> v;
        for(size_t d = start; d < p.rank; ++d)
            v.push_back({p.lengths[d], p.outputLengths[d], p.desc.inStrides[d], p.desc.outStrides[d]});
        if(v.empty())
            return;
        auto by_in = [](const IoDim& a, const IoDim& b) {
            if(a.len == 1 && b.len != 1)
                return false;
            if(b.len == 1 && a.len != 1)
                return true;
            return a.is < b.is;
        };
        auto by_out = [](const IoDim& a, const IoDim& b) {
            if(a.len == 1 && b.len != 1)
                return false;
            if(b.len == 1 && a.len != 1)
                return true;
            return a.os < b.os;
        };
        std::stable_sort(v.begin(), v.end(), by_in);
        if(!std::is_sorted(v.begin(), v.end(), by_out))
            return; // a transposing layout: leave the caller's order alone
        while(v.size() > 1 && v.back().len == 1)
        {
            --p.rank;
            v.pop_back();
        }
        p.lengths.resize(p.rank);
        p.outputLengths.resize(p.rank);
        p.desc.inStrides.resize(p.rank);
        p.desc.outStrides.resize(p.rank);
        for(size_t d = start; d < p.rank; ++d)
        {
            p.lengths[d]         = v[d - start].len;
            p.outputLengths[d]   = v[d - start].olen;
            p.desc.inStrides[d]  = v[d - start].is;
            p.desc.outStrides[d] = v[d - start].os;
        }
    }

    // plan.cpp:729-779 in the reference
    rocfft_status check_array_types(const rocfft_plan_t& p)
    {
        const auto in = p.desc.inArrayType, out = p.desc.outArrayType;
        const bool ip = p.placement == rocfft_placement_inplace;
        switch(p.transformType)
        {
        case rocfft_transform_type_complex_forward:
        case rocfft_transform_type_complex_inverse:
            if(in != rocfft_array_type_complex_interleaved && in != rocfft_array_type_complex_planar)
                return rocfft_status_invalid_array_type;
            if(out != rocfft_array_type_complex_interleaved && out != rocfft_array_type_complex_planar)
                return rocfft_status_invalid_array_type;
            if(ip && in != out)
                return rocfft_status_invalid_array_type;
            break;
        case rocfft_transform_type_real_forward:
            if(in != rocfft_array_type_real)
                return rocfft_status_invalid_array_type;
            if(out != rocfft_array_type_hermitian_interleaved && out != rocfft_array_type_hermitian_planar)
                return rocfft_status_invalid_array_type;
            if(ip && out != rocfft_array_type_hermitian_interleaved)
                return rocfft_status_invalid_array_type;
            break;
        case rocfft_transform_type_real_inverse:
            if(out != rocfft_array_type_real)
                return rocfft_status_invalid_array_type;
            if(in != rocfft_array_type_hermitian_interleaved && in != rocfft_array_type_hermitian_planar)
                return rocfft_status_invalid_array_type;
            if(ip && in != rocfft_array_type_hermitian_interleaved)
                return rocfft_status_invalid_array_type;
            break;
        }
        return rocfft_status_success;
    }
}

extern "C" {

rocfft_status rocfft_setup()
{
    log().init();
    log_trace(__func__);
    return rocfft_status_success;
}

rocfft_status rocfft_cleanup()
{
    log_trace(__func__);
    return rocfft_status_success;
}

rocfft_status rocfft_plan_description_create(rocfft_plan_description* description)
{
    if(!description)
        return rocfft_status_failure;
    *description = new rocfft_plan_description_t;
    log_trace(__func__, "description", (void*)*description);
    return rocfft_status_success;
}

rocfft_status rocfft_plan_description_destroy(rocfft_plan_description description)
{
    log_trace(__func__, "description", (void*)description);
    delete description;
    return rocfft_status_success;
}

rocfft_status rocfft_plan_description_set_scale_factor(rocfft_plan_description description,
                                                       const double            scale_factor)
{
    log_trace(__func__, "description", (void*)description, "scale", scale_factor);
    if(!description)
        return rocfft_status_failure;
    if(!std::isfinite(scale_factor))
        return rocfft_status_invalid_arg_value;
    description->scale = scale_factor;
    return rocfft_status_success;
}

rocfft_status rocfft_plan_description_set_data_layout(rocfft_plan_description description,
                                                      const rocfft_array_type in_array_type,
                                                      const rocfft_array_type out_array_type,
                                                      const size_t*           in_offsets,
                                                      const size_t*           out_offsets,
                                                      const size_t            in_strides_size,
                                                      const size_t*           in_strides,
                                                      const size_t            in_distance,
                                                      const size_t            out_strides_size,
                                                      const size_t*           out_strides,
                                                      const size_t            out_distance)
{
    log_trace(__func__,
              "description",
              (void*)description,
              "in_array_type",
              (int)in_array_type,
              "out_array_type",
              (int)out_array_type,
              "in_distance",
              in_distance,
              "out_distance",
              out_distance);
    if(!description)
        return rocfft_status_failure;
    description->inArrayType  = in_array_type;
    description->outArrayType = out_array_type;
    if(in_offsets)
        for(size_t i = 0; i < offset_count(in_array_type); ++i)
            description->inOffset[i] = in_offsets[i];
    if(out_offsets)
        for(size_t i = 0; i < offset_count(out_array_type); ++i)
            description->outOffset[i] = out_offsets[i];
    if(in_strides)
        description->inStrides.assign(in_strides, in_strides + in_strides_size);
    if(in_distance)
        description->inDist = in_distance;
    if(out_strides)
        description->outStrides.assign(out_strides, out_strides + out_strides_size);
    if(out_distance)
        description->outDist = out_distance;
    return rocfft_status_success;
}

rocfft_status rocfft_plan_description_set_comm(rocfft_plan_description description,
                                               rocfft_comm_type        comm_type,
                                               void*                   comm_handle)
{
    log_trace(__func__, "description", (void*)description, "comm_type", (int)comm_type);
    if(!description)
        return rocfft_status_failure;
    if(comm_type == rocfft_comm_mpi)
        return rocfft_status_invalid_arg_value; // this build exchanges data with NCCL, not MPI
    if(comm_type == rocfft_comm_nccl && !comm_handle)
        return rocfft_status_invalid_arg_value;
    description->comm_type   = comm_type;
    description->comm_handle = comm_handle;
    return rocfft_status_success;
}

rocfft_status rocfft_field_create(rocfft_field* field)
{
    if(!field)
        return rocfft_status_failure;
    *field = new rocfft_field_t;
    return rocfft_status_success;
}

rocfft_status rocfft_field_destroy(rocfft_field field)
{
    delete field;
    return rocfft_status_success;
}

rocfft_status rocfft_brick_create(rocfft_brick* brick,
                                  const size_t* field_lower,
                                  const size_t* field_upper,
                                  const size_t* brick_stride,
                                  size_t        dim,
                                  int           deviceID)
{
    if(!brick || !field_lower || !field_upper || !brick_stride || dim < 2 || dim > 4)
        return rocfft_status_invalid_arg_value;
    for(size_t i = 0; i < dim; ++i)
        if(field_lower[i] >= field_upper[i])
            return rocfft_status_invalid_dimensions;
    auto* b = new rocfft_brick_t;
    b->lower.assign(field_lower, field_lower + dim);
    b->upper.assign(field_upper, field_upper + dim);
    b->stride.assign(brick_stride, brick_stride + dim);
    b->device = deviceID;
    *brick    = b;
    return rocfft_status_success;
}

rocfft_status rocfft_brick_destroy(rocfft_brick brick)
{
    delete brick;
    return rocfft_status_success;
}

rocfft_status rocfft_field_add_brick(rocfft_field field, rocfft_brick brick)
{
    if(!field || !brick)
        return rocfft_status_invalid_arg_value;
    field->bricks.push_back(*brick);
    return rocfft_status_success;
}

rocfft_status rocfft_plan_description_add_infield(rocfft_plan_description description, rocfft_field field)
{
    if(!description || !field)
        return rocfft_status_invalid_arg_value;
    description->inFields.push_back(*field);
    return rocfft_status_success;
}

rocfft_status rocfft_plan_description_add_outfield(rocfft_plan_description description, rocfft_field field)
{
    if(!description || !field)
        return rocfft_status_invalid_arg_value;
    description->outFields.push_back(*field);
    return rocfft_status_success;
}

rocfft_status rocfft_plan_create(rocfft_plan*                  plan,
                                 rocfft_result_placement       placement,
                                 rocfft_transform_type         transform_type,
                                 rocfft_precision              precision,
                                 size_t                        dimensions,
                                 const size_t*                 lengths,
                                 size_t                        number_of_transforms,
                                 const rocfft_plan_description description)
{
    if(!plan)
        return rocfft_status_failure;
    rocfft_plan_t* p = new rocfft_plan_t;
    *plan            = p; // like the reference, the handle exists even when creation fails
    log_trace(__func__,
              "plan",
              (void*)p,
              "placement",
              (int)placement,
              "transform_type",
              (int)transform_type,
              "precision",
              (int)precision,
              "dimensions",
              dimensions,
              "number_of_transforms",
              number_of_transforms,
              "description",
              (void*)description);
    if(dimensions > 3)
        return rocfft_status_invalid_dimensions;
    if(dimensions == 0 || !lengths)
        return rocfft_status_invalid_dimensions;
    try
    {
        for(size_t i = 0; i < dimensions; ++i)
            if(lengths[i] == 0)
                return rocfft_status_invalid_dimensions;
        p->rank = dimensions;
        p->lengths.assign(lengths, lengths + dimensions);
        p->userLengths = p->lengths;
        p->batch         = number_of_transforms;
        p->placement     = placement;
        p->precision     = precision;
        p->transformType = transform_type;
        p->outputLengths = p->lengths;
        const bool real  = transform_type == rocfft_transform_type_real_forward
                          || transform_type == rocfft_transform_type_real_inverse;
        if(real)
            p->outputLengths[0] = p->outputLengths[0] / 2 + 1;
        if(transform_type == rocfft_transform_type_real_inverse)
            std::swap(p->outputLengths, p->lengths);
        if(description)
            p->desc = *description;
        if((!p->desc.inStrides.empty() && p->desc.inStrides.size() != dimensions)
           || (!p->desc.outStrides.empty() && p->desc.outStrides.size() != dimensions))
            return rocfft_status_invalid_strides;
        init_defaults(p->desc, transform_type, placement, p->lengths, p->outputLengths);
        if(log().layer & 2)
        {
            std::lock_guard<std::mutex> g(log().mtx);
            log().bench() << bench_command(*p) << std::endl;
        }
        sort_dims(*p);
        rocfft_status st = check_array_types(*p);
        if(st != rocfft_status_success)
            return st;
        if(!p->desc.inFields.empty() || !p->desc.outFields.empty())
            b200fft::build_multi_device_plan(p);
        else
            b200fft::build_single_device_plan(p);

        if(log().layer & 8)
        {
            std::lock_guard<std::mutex> g(log().mtx);
            if(p->core)
                log().plan() << b200fft::describe_core(*p->core) << std::endl;
        }
        if((log().layer & 128) && p->mgpu)
        {
            // graph layer: the multi-device plan as a graphviz digraph (reference: library/src/transform.cpp:178-254)
            std::lock_guard<std::mutex> g(log().mtx);
            log().graph() << b200fft::multi_device_plan_graph(p) << std::endl;
        }
        return rocfft_status_success;
    }
    catch(rocfft_status s)
    {
        return s;
    }
    catch(std::exception& e)
    {
        log_trace("rocfft_plan_create failed", e.what());
        if(getenv("B200FFT_DEBUG"))
            fprintf(stderr, "rocfft_plan_create: %s\n", e.what());
        return rocfft_status_failure;
    }
}

rocfft_status rocfft_plan_destroy(rocfft_plan plan)
{
    log_trace(__func__, "plan", (void*)plan);
    if(plan)
    {
        b200fft::destroy_multi_device_plan(plan);
        delete plan;
    }
    return rocfft_status_success;
}

rocfft_status rocfft_plan_get_work_buffer_size(const rocfft_plan plan, size_t* size_in_bytes)
{
    if(!plan || !size_in_bytes)
        return rocfft_status_failure;
    *size_in_bytes = plan->core ? plan->core->work_bytes : 0;
    if(plan->mgpu)
        *size_in_bytes = b200fft::multi_device_work_bytes(plan);
    log_trace(__func__, "plan", (void*)plan, "val", *size_in_bytes);
    return rocfft_status_success;
}

rocfft_status rocfft_plan_get_print(const rocfft_plan plan)
{
    log_trace(__func__, "plan", (void*)plan);
    if(!plan)
        return rocfft_status_failure;
    std::cout << "rank: " << plan->rank << "\nlengths:";
    for(size_t l : plan->lengths)
        std::cout << " " << l;
    std::cout << "\nbatch: " << plan->batch << "\n";
    if(plan->core)
        std::cout << b200fft::describe_core(*plan->core);
    std::cout << std::endl;
    return rocfft_status_success;
}

rocfft_status rocfft_get_version_string(char* buf, size_t len)
{
    static const char v[] = B200FFT_VERSION_STRING;
    if(!buf)
        return rocfft_status_failure;
    if(len < sizeof(v))
        return rocfft_status_invalid_arg_value;
    memcpy(buf, v, sizeof(v));
    return rocfft_status_success;
}

rocfft_status rocfft_execution_info_create(rocfft_execution_info* info)
{
    if(!info)
        return rocfft_status_failure;
    *info = new rocfft_execution_info_t;
    log_trace(__func__, "info", (void*)*info);
    return rocfft_status_success;
}

rocfft_status rocfft_execution_info_destroy(rocfft_execution_info info)
{
    log_trace(__func__, "info", (void*)info);
    delete info;
    return rocfft_status_success;
}

rocfft_status rocfft_execution_info_set_work_buffer(rocfft_execution_info info,
                                                    void*                 work_buffer,
                                                    const size_t          size_in_bytes)
{
    log_trace(__func__, "info", (void*)info, "work_buffer", work_buffer, "size_in_bytes", size_in_bytes);
    if(!info)
        return rocfft_status_failure;
    if(!work_buffer)
        return rocfft_status_invalid_work_buffer;
    info->workBuffer     = work_buffer;
    info->workBufferSize = size_in_bytes;
    return rocfft_status_success;
}

rocfft_status rocfft_execution_info_set_stream(rocfft_execution_info info, void* stream)
{
    log_trace(__func__, "info", (void*)info, "stream", stream);
    if(!info)
        return rocfft_status_failure;
    info->stream = (cudaStream_t)stream;
    return rocfft_status_success;
}

rocfft_status rocfft_execution_info_set_load_callback(rocfft_execution_info info,
                                                      void**                cb_functions,
                                                      void**                cb_data,
                                                      size_t                shared_mem_bytes)
{
    (void)cb_data;
    if(!info)
        return rocfft_status_failure;
    if(shared_mem_bytes)
        return rocfft_status_invalid_arg_value;
    info->load_cb = cb_functions ? cb_functions[0] : nullptr;
    return rocfft_status_success;
}

rocfft_status rocfft_execution_info_set_store_callback(rocfft_execution_info info,
                                                       void**                cb_functions,
                                                       void**                cb_data,
                                                       size_t                shared_mem_bytes)
{
    (void)cb_data;
    if(!info)
        return rocfft_status_failure;
    if(shared_mem_bytes)
        return rocfft_status_invalid_arg_value;
    info->store_cb = cb_functions ? cb_functions[0] : nullptr;
    return rocfft_status_success;
}

rocfft_status rocfft_execute(const rocfft_plan     plan,
                             void*                 in_buffer[],
                             void*                 out_buffer[],
                             rocfft_execution_info info)
{
    log_trace(__func__, "plan", (void*)plan, "in", (void*)in_buffer, "out", (void*)out_buffer, "info", (void*)info);
    if(!plan || !in_buffer)
        return rocfft_status_failure;
    try
    {
        rocfft_execution_info_t ei;
        if(info)
            ei = *info;
        if(ei.load_cb || ei.store_cb)
            return rocfft_status_failure; // user callbacks are not implemented
        if(plan->mgpu)
            return b200fft::execute_multi_device_plan(plan, in_buffer, out_buffer, &ei);
        if(!plan->core)
            return rocfft_status_failure;
        const b200fft::PlanCore& core = *plan->core;

        void* work      = nullptr;
        bool  own_alloc = false;
        if(core.work_bytes > 0)
        {
            if(ei.workBuffer)
            {
                if(ei.workBufferSize < core.work_bytes)
                    return rocfft_status_invalid_work_buffer;
                work = ei.workBuffer;
            }
            else
            {
                // stream-ordered allocation: freed on the same stream after the last step
                if(cudaMallocAsync(&work, core.work_bytes, ei.stream) != cudaSuccess)
                    return rocfft_status_failure;
                own_alloc = true;
            }
        }
        if(log().layer & 4)
        {
            // profile layer: time every kernel with events, wait, report (this synchronises the stream)
            const size_t             n = core.steps.size();
            std::vector<cudaEvent_t> ev(n + 1);
            for(auto& e : ev)
                cudaEventCreate(&e);
            rocfft_status st = b200fft::execute_core(core, in_buffer, out_buffer, work, ei.stream, ev.data());
            if(own_alloc)
                cudaFreeAsync(work, ei.stream);
            cudaStreamSynchronize(ei.stream);
            const double peak = max_memory_bandwidth_gbs();
            for(size_t i = 0; i < n; ++i)
            {
                float ms = 0.f;
                cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
                const b200fft::Step& sp    = core.steps[i];
                unsigned long long   elems = 0;
                if(sp.kind == b200fft::Step::TILE && sp.kern)
                {
                    elems = (unsigned long long)sp.kern->length * sp.ka.on[0] * sp.ka.on[1] * sp.ka.on[2];
                    for(const auto& l : sp.loops)
                        elems *= l.count;
                }
                const unsigned long long bytes = elems * (sp.in_elem_bytes + sp.out_elem_bytes);
                const double             gbs   = ms > 0 ? bytes / (ms * 1e6) : 0.0;
                std::lock_guard<std::mutex> g(log().mtx);
                log().profile() << "rocfft_execute,scheme," << sp.note << ",duration_ms," << ms << ",total_size_bytes,"
                                << bytes << ",exec_GB_s," << gbs << ",max_mem_GB_s," << peak << ",bw_efficiency_pct,"
                                << (peak > 0 ? 100.0 * gbs / peak : 0.0) << ",kernel_index," << i << std::endl;
            }
            for(auto& e : ev)
                cudaEventDestroy(e);
            return st;
        }
        if(log().layer & 16)
        {
            // kernelio layer: a checksum of what every kernel left in its output buffer (this synchronises the stream).
            // The reference dumps and hashes each kernel's input and output (library/src/powX.cpp:743-780, 910-956);
            // here one order-independent 64-bit sum per kernel over the extent of its output view is written, which is
            // what run-to-run comparisons need.
            struct Ctx
            {
                unsigned long long* dev;
                size_t              n;
                std::vector<size_t> bytes;
            } ctx{nullptr, core.steps.size(), std::vector<size_t>(core.steps.size(), 0)};
            if(cudaMalloc(&ctx.dev, sizeof(unsigned long long) * std::max<size_t>(ctx.n, 1)) != cudaSuccess)
                return rocfft_status_failure;
            auto obs = [](void* c, size_t i, const b200fft::Step& sp, void* out_ptr, cudaStream_t s) {
                Ctx* x = static_cast<Ctx*>(c);
                if(i >= x->n || !out_ptr)
                    return;
                // extent of the output view in elements: 1 + sum (len - 1) * |stride| over the kernel's dimensions
                const bool tile = sp.kind != b200fft::Step::EW;
                const b200fft_ioview& v = tile ? sp.ka.out : sp.ea.out;
                const unsigned*       on = tile ? sp.ka.on : sp.ea.on;
                unsigned long long n0 = tile ? (sp.kern ? (unsigned long long)sp.kern->length : 1) : sp.ea.n;
                if(tile && sp.kern && sp.kern->variant == B200FFT_2D_L2)
                    n0 = (unsigned long long)sp.ka.on[0] * sp.ka.on[0];
                if(v.blk >= 2 || v.planar)
                    return; // per-rank blocks and planar outputs are not one byte range
                unsigned long long el = 1 + (n0 ? n0 - 1 : 0) * (unsigned long long)std::llabs(v.es);
                for(int k = 0; k < 3; ++k)
                    el += (unsigned long long)(on[k] ? on[k] - 1 : 0) * (unsigned long long)std::llabs(v.os[k]);
                for(const auto& l : sp.loops)
                    el += (unsigned long long)(l.count ? l.count - 1 : 0) * (unsigned long long)std::llabs(l.out_stride);
                x->bytes[i] = (size_t)el * sp.out_elem_bytes;
                b200fft_launch_hash(out_ptr, x->bytes[i], x->dev + i, s);
            };
            rocfft_status st = b200fft::execute_core(core, in_buffer, out_buffer, work, ei.stream, nullptr, obs, &ctx);
            if(own_alloc)
                cudaFreeAsync(work, ei.stream);
            cudaStreamSynchronize(ei.stream);
            std::vector<unsigned long long> h(std::max<size_t>(ctx.n, 1), 0);
            cudaMemcpy(h.data(), ctx.dev, sizeof(unsigned long long) * ctx.n, cudaMemcpyDeviceToHost);
            cudaFree(ctx.dev);
            std::lock_guard<std::mutex> g(log().mtx);
            for(size_t i = 0; i < ctx.n; ++i)
            {
                log().kernelio() << "--- --- kernel " << i << " (" << core.steps[i].note << ") output: ";
                if(ctx.bytes[i])
                    log().kernelio() << ctx.bytes[i] << " bytes, hash " << std::hex << h[i] << std::dec << std::endl;
                else
                    log().kernelio() << "not hashed (blocked or planar layout)" << std::endl;
            }
            return st;
        }
        rocfft_status st = b200fft::execute_core(core, in_buffer, out_buffer, work, ei.stream);
        if(own_alloc)
            cudaFreeAsync(work, ei.stream);
        return st;
    }
    catch(rocfft_status s)
    {
        return s;
    }
    catch(std::exception&)
    {
        return rocfft_status_failure;
    }
}

// ---- extensions (include/rocfft_b200_ext.h) ----
ROCFFT_EXPORT rocfft_status b200fft_plan_describe(const rocfft_plan plan, char* buf, size_t len)
{
    if(!plan || !buf || !len)
        return rocfft_status_failure;
    std::string s = plan->core ? b200fft::describe_core(*plan->core) : std::string("multi-device plan\n");
    if(plan->mgpu)
        s = b200fft::describe_multi_device_plan(plan);
    if(s.size() + 1 > len)
        s.resize(len - 1);
    memcpy(buf, s.c_str(), s.size() + 1);
    return rocfft_status_success;
}

ROCFFT_EXPORT rocfft_status b200fft_plan_device_error(const rocfft_plan plan, int* raised)
{
    if(!plan || !raised)
        return rocfft_status_failure;
    std::vector<const int*> flags;
    if(plan->core && plan->core->dev_error)
        flags.push_back(plan->core->dev_error);
    if(plan->mgpu)
        b200fft::multi_device_error_flags(plan, flags);
    *raised = 0;
    for(const int* f : flags)
    {
        int v = 0;
        if(cudaMemcpy(&v, f, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
            return rocfft_status_failure;
        *raised |= (v != 0);
    }
    return rocfft_status_success;
}

ROCFFT_EXPORT rocfft_status b200fft_slab_exchange_offsets(int     ranks,
                                                          int     chunks,
                                                          size_t  slab_bytes,
                                                          int     first,
                                                          int     chunk,
                                                          size_t* send_off,
                                                          size_t* recv_off,
                                                          size_t* block_bytes)
{
    if(ranks < 1 || chunks < 1 || chunk < 0 || chunk >= chunks || !send_off || !recv_off || !block_bytes)
        return rocfft_status_invalid_arg_value;
    b200fft::slab_exchange_offsets(ranks, chunks, slab_bytes, first, chunk, send_off, recv_off, block_bytes);
    return rocfft_status_success;
}

ROCFFT_EXPORT rocfft_status b200fft_rows2d_exchange_offsets(
    int ranks, int rank, size_t nx, size_t ny, size_t elem_bytes, size_t* first_off, size_t* second_off)
{
    if(ranks < 1 || rank < 0 || rank >= ranks || !first_off || !second_off || nx % (size_t)ranks || ny % (size_t)ranks)
        return rocfft_status_invalid_arg_value;
    b200fft::rows2d_exchange_offsets(ranks, rank, nx, ny, elem_bytes, first_off, second_off);
    return rocfft_status_success;
}

ROCFFT_EXPORT rocfft_status b200fft_nccl_unique_id(void* id128)
{
    return b200fft::nccl_unique_id(id128) == 0 ? rocfft_status_success : rocfft_status_failure;
}
ROCFFT_EXPORT rocfft_status b200fft_nccl_comm_create(int nranks, int rank, const void* id128, void** comm)
{
    if(!id128 || !comm)
        return rocfft_status_invalid_arg_value;
    return b200fft::nccl_comm_create(nranks, rank, id128, comm) == 0 ? rocfft_status_success : rocfft_status_failure;
}
ROCFFT_EXPORT rocfft_status b200fft_nccl_comm_destroy(void* comm)
{
    return b200fft::nccl_comm_destroy(comm) == 0 ? rocfft_status_success : rocfft_status_failure;
}

ROCFFT_EXPORT unsigned long long b200fft_launch_count()
{
    return b200fft::g_launch_count.load();
}

// Executes the plan once with an event between consecutive steps and reports
// each step's device time; synchronises the stream (profiling only).
ROCFFT_EXPORT rocfft_status b200fft_execute_profiled(const rocfft_plan     plan,
                                                     void*                 in_buffer[],
                                                     void*                 out_buffer[],
                                                     rocfft_execution_info info,
                                                     float*                step_ms,
                                                     size_t                max_steps,
                                                     size_t*               nsteps)
{
    if(!plan || !plan->core || !in_buffer || !step_ms || !nsteps)
        return rocfft_status_failure;
    const b200fft::PlanCore& core = *plan->core;
    rocfft_execution_info_t  ei;
    if(info)
        ei = *info;
    if(core.work_bytes > 0 && (!ei.workBuffer || ei.workBufferSize < core.work_bytes))
        return rocfft_status_invalid_work_buffer;
    const size_t             n = core.steps.size();
    std::vector<cudaEvent_t> ev(n + 1);
    for(auto& e : ev)
        cudaEventCreate(&e);
    rocfft_status st = b200fft::execute_core(core, in_buffer, out_buffer, ei.workBuffer, ei.stream, ev.data());
    cudaStreamSynchronize(ei.stream);
    *nsteps = n;
    for(size_t i = 0; i < n && i < max_steps; ++i)
        cudaEventElapsedTime(&step_ms[i], ev[i], ev[i + 1]);
    for(auto& e : ev)
        cudaEventDestroy(e);
    return st;
}

ROCFFT_EXPORT rocfft_status b200fft_stacked_twiddles(
    int n, const int* factors, int nfactors, int precision, void* out, size_t out_bytes, size_t* needed)
{
    std::vector<char> h;
    b200fft::host_stacked_twiddles(n, factors, nfactors, precision, h);
    if(needed)
        *needed = h.size();
    if(out && out_bytes >= h.size())
        memcpy(out, h.data(), h.size());
    return rocfft_status_success;
}

ROCFFT_EXPORT rocfft_status b200fft_pool_query(size_t index, int* length, int* precision, int* variant, int* factors8, size_t* count)
{
    size_t                    cnt = 0;
    const b200fft_pool_entry* p   = b200fft_pool(&cnt);
    if(count)
        *count = cnt;
    if(index >= cnt)
        return rocfft_status_invalid_arg_value;
    if(length)
        *length = p[index].length;
    if(precision)
        *precision = p[index].precision;
    if(variant)
        *variant = p[index].variant;
    if(factors8)
        for(int i = 0; i < 8; ++i)
            factors8[i] = p[index].factors[i];
    return rocfft_status_success;
}

rocfft_status rocfft_cache_serialize(void** buffer, size_t* buffer_len_bytes)
{
    if(!buffer || !buffer_len_bytes)
        return rocfft_status_invalid_arg_value;
    *buffer           = malloc(1);
    *buffer_len_bytes = 0;
    return rocfft_status_success;
}

rocfft_status rocfft_cache_buffer_free(void* buffer)
{
    free(buffer);
    return rocfft_status_success;
}

rocfft_status rocfft_cache_deserialize(const void* buffer, size_t buffer_len_bytes)
{
    (void)buffer_len_bytes;
    if(!buffer)
        return rocfft_status_invalid_arg_value;
    return rocfft_status_success;
}

} // extern "C"
