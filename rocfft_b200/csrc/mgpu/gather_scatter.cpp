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
//
// Across processes (rocfft_comm_nccl; each rank adds its own bricks, as the ranks of
// clients/samples/mpi/rocfft_mpi_example.cpp do) the same plan serves every layout
// the slab plan does not take — other ranks, uneven slabs, several bricks per rank,
// real transforms: the ranks all-gather their brick boxes at plan creation, rank 0
// owns the gathered field and the single-device plan, the other ranks pack their
// bricks into a contiguous staging buffer and ncclSend them (rank 0: ncclRecv, then
// unpack), and the result travels back the same way.
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
            std::vector<BoxCopy> gathers, scatters; // this rank's own bricks
            // multi-process mode
            ncclComm_t comm = nullptr;
            int        P = 1, rank = 0;
            struct Remote
            {
                int     owner;
                BoxCopy box; // brick_stride = contiguous packing of the box
                size_t  staging_off, bytes;
            };
            std::vector<Remote> remote_in, remote_out; // rank 0: every other rank's bricks, by rank then order
            std::vector<Remote> mine_in, mine_out; // other ranks: own bricks as they travel
            void*               staging = nullptr;
            size_t              staging_bytes = 0;
        };

        constexpr int MAXB = 8; // bricks per rank and field in multi-process plans
        struct RankBricks
        {
            unsigned long long n_in, n_out;
            unsigned long long in_lo[MAXB][4], in_hi[MAXB][4], out_lo[MAXB][4], out_hi[MAXB][4];
        };

        // all-gather of one fixed-size record per rank (collective; uses the default stream)
        template <class R>
        std::vector<R> allgather_records(ncclComm_t comm, int P, const R& mine)
        {
            NcclApi& N    = nccl();
            char*    dbuf = nullptr;
            if(cudaMalloc(&dbuf, sizeof(R) * (P + 1)) != cudaSuccess)
                throw std::runtime_error("cudaMalloc failed");
            cudaMemcpy(dbuf, &mine, sizeof(R), cudaMemcpyHostToDevice);
            ncclResult_t   r = N.AllGather(dbuf, dbuf + sizeof(R), sizeof(R), ncclChar, comm, nullptr);
            cudaError_t    e = cudaStreamSynchronize(nullptr);
            std::vector<R> all(P);
            cudaMemcpy(all.data(), dbuf + sizeof(R), sizeof(R) * P, cudaMemcpyDeviceToHost);
            cudaFree(dbuf);
            if(r != ncclSuccess || e != cudaSuccess)
                throw std::runtime_error("brick exchange between ranks failed");
            return all;
        }

        void contiguous_box(BoxCopy& c)
        {
            long long s = 1;
            for(int i = 0; i < 4; ++i)
            {
                c.brick_stride[i] = s;
                s *= (long long)c.n[i];
            }
        }
        size_t box_count(const BoxCopy& c)
        {
            return (size_t)(c.n[0] * c.n[1] * c.n[2] * c.n[3]);
        }

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
        const size_t dim           = in_len.size();
        const bool   outer_inplace = plan->placement == rocfft_placement_inplace;
        if(outer_inplace && d.inFields[0].bricks.size() != d.outFields[0].bricks.size())
            throw std::runtime_error("in-place plans need as many output bricks as input bricks");

        auto gp         = std::make_unique<GatherPlan>();
        const bool multi = d.comm_type == rocfft_comm_nccl;
        std::vector<RankBricks> all; // multi-process: every rank's boxes
        if(!multi)
        {
            validate_field(d.inFields[0], in_len);
            validate_field(d.outFields[0], out_len);
        }
        else
        {
            NcclApi& N = nccl();
            if(!N.ok || !d.comm_handle)
                throw std::runtime_error("multi-process plans need libnccl and a communicator");
            gp->comm = *static_cast<ncclComm_t*>(d.comm_handle);
            if(N.CommCount(gp->comm, &gp->P) != ncclSuccess || N.CommUserRank(gp->comm, &gp->rank) != ncclSuccess)
                throw std::runtime_error("NCCL communicator query failed");
            // a rank whose own bricks are malformed still takes part in the exchange (with a marker),
            // so that every rank fails together instead of one of them waiting forever
            RankBricks mine{};
            bool       local_ok = d.inFields[0].bricks.size() <= (size_t)MAXB
                            && d.outFields[0].bricks.size() <= (size_t)MAXB && !d.inFields[0].bricks.empty()
                            && !d.outFields[0].bricks.empty();
            auto pack = [&](const rocfft_field_t& f, unsigned long long& n, unsigned long long (*lo)[4],
                            unsigned long long (*hi)[4]) {
                n = f.bricks.size();
                for(size_t b = 0; b < f.bricks.size() && local_ok; ++b)
                {
                    const auto& br = f.bricks[b];
                    if(br.lower.size() != dim || br.upper.size() != dim || br.stride.size() != dim)
                    {
                        local_ok = false;
                        break;
                    }
                    for(size_t i = 0; i < 4; ++i)
                    {
                        lo[b][i] = i < dim ? br.lower[i] : 0;
                        hi[b][i] = i < dim ? br.upper[i] : 1;
                    }
                }
            };
            if(local_ok)
            {
                pack(d.inFields[0], mine.n_in, mine.in_lo, mine.in_hi);
                pack(d.outFields[0], mine.n_out, mine.out_lo, mine.out_hi);
            }
            if(!local_ok)
                mine.n_in = mine.n_out = ~0ull;
            all = allgather_records(gp->comm, gp->P, mine);
            rocfft_field_t gin, gout;
            for(int q = 0; q < gp->P; ++q)
            {
                if(all[q].n_in == ~0ull)
                    throw std::runtime_error("a rank supplied malformed bricks");
                auto unpack = [&](unsigned long long n, unsigned long long (*lo)[4], unsigned long long (*hi)[4],
                                  rocfft_field_t& f) {
                    for(unsigned long long b = 0; b < n; ++b)
                    {
                        rocfft_brick_t br;
                        br.lower.assign(lo[b], lo[b] + dim);
                        br.upper.assign(hi[b], hi[b] + dim);
                        br.stride.assign(dim, 1);
                        br.rank = q;
                        f.bricks.push_back(br);
                    }
                };
                unpack(all[q].n_in, all[q].in_lo, all[q].in_hi, gin);
                unpack(all[q].n_out, all[q].out_lo, all[q].out_hi, gout);
            }
            validate_field(gin, in_len);
            validate_field(gout, out_len);
        }

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
        const bool owner = !multi || gp->rank == 0; // holds the gathered field and the single-device plan

        if(multi)
        {
            // boxes as they travel: contiguous in the staging buffer on both ends
            auto travel = [&](const std::vector<BoxCopy>& own, int elem, std::vector<GatherPlan::Remote>& out) {
                size_t off = 0;
                for(const BoxCopy& c : own)
                {
                    GatherPlan::Remote r;
                    r.owner = gp->rank;
                    r.box   = c;
                    // staging side takes the place of the full array: contiguous, no offset
                    long long s = 1;
                    for(int i = 0; i < 4; ++i)
                    {
                        r.box.full_stride[i] = s;
                        s *= (long long)c.n[i];
                    }
                    r.box.full_offset = 0;
                    r.staging_off     = off;
                    r.bytes           = box_count(c) * (size_t)elem;
                    off += (r.bytes + 255) & ~size_t(255);
                    out.push_back(r);
                }
                return off;
            };
            auto remote = [&](bool input, const std::vector<size_t>& len, int elem, std::vector<GatherPlan::Remote>& out) {
                size_t off = 0;
                for(int q = 1; q < gp->P; ++q)
                {
                    rocfft_field_t f;
                    const auto     n = input ? all[q].n_in : all[q].n_out;
                    for(unsigned long long b = 0; b < n; ++b)
                    {
                        rocfft_brick_t br;
                        auto*          lo = input ? all[q].in_lo[b] : all[q].out_lo[b];
                        auto*          hi = input ? all[q].in_hi[b] : all[q].out_hi[b];
                        br.lower.assign(lo, lo + dim);
                        br.upper.assign(hi, hi + dim);
                        br.stride.assign(dim, 1);
                        f.bricks.push_back(br);
                    }
                    std::vector<BoxCopy> boxes;
                    make_copies(f, len, boxes);
                    for(BoxCopy& c : boxes)
                    {
                        contiguous_box(c); // the brick side is the packed staging copy
                        GatherPlan::Remote r;
                        r.owner       = q;
                        r.box         = c;
                        r.staging_off = off;
                        r.bytes       = box_count(c) * (size_t)elem;
                        off += (r.bytes + 255) & ~size_t(255);
                        out.push_back(r);
                    }
                }
                return off;
            };
            if(gp->rank == 0)
                gp->staging_bytes = std::max(remote(true, in_len, gp->in_elem, gp->remote_in),
                                             remote(false, out_len, gp->out_elem, gp->remote_out));
            else
                gp->staging_bytes = std::max(travel(gp->gathers, gp->in_elem, gp->mine_in),
                                             travel(gp->scatters, gp->out_elem, gp->mine_out));
        }

        // the single-device plan on contiguous arrays
        bool created = true;
        if(owner)
        {
            rocfft_plan_description desc = nullptr;
            rocfft_status           st   = rocfft_plan_description_create(&desc);
            if(st == rocfft_status_success)
                st = rocfft_plan_description_set_data_layout(
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
            created = st == rocfft_status_success;
        }

        int ndev = 0;
        if(cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
        {
            cudaGetLastError();
            gp->host_only = true; // inspectable only
        }
        else if(created)
        {
            cudaGetDevice(&gp->device);
            if(!multi)
                for(auto* v : {&gp->gathers, &gp->scatters})
                    for(const BoxCopy& c : *v)
                    {
                        if(c.device < 0 || c.device >= ndev)
                        {
                            created = false;
                            break;
                        }
                        if(c.device == gp->device)
                            continue;
                        gp->remote = true;
                        int ok     = 0;
                        cudaDeviceCanAccessPeer(&ok, gp->device, c.device);
                        const cudaError_t e = ok ? cudaDeviceEnablePeerAccess(c.device, 0) : cudaErrorInvalidDevice;
                        cudaGetLastError();
                        if(e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                        {
                            created = false;
                            break;
                        }
                    }
            if(created && owner)
            {
                created = cudaMalloc(&gp->full_in, gp->in_bytes) == cudaSuccess
                          && (gp->inplace || cudaMalloc(&gp->full_out, gp->out_bytes) == cudaSuccess);
                if(gp->inplace)
                    gp->full_out = gp->full_in;
            }
            if(created && gp->staging_bytes)
                created = cudaMalloc(&gp->staging, gp->staging_bytes) == cudaSuccess;
        }
        if(multi && !gp->host_only)
        {
            // every rank learns whether every rank got its resources
            struct Flag
            {
                int ok;
            } f{created ? 1 : 0};
            for(const Flag& o : allgather_records(gp->comm, gp->P, f))
                created = created && o.ok;
        }
        plan->mgpu = gp.release();
        if(!created)
        {
            destroy_gather_scatter_plan(plan);
            throw std::runtime_error("gather/scatter plan: the single-device plan, peer access or an allocation failed");
        }
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
        if(gp->staging)
            cudaFree(gp->staging);
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
        if(!gp || gp->host_only)
            return rocfft_status_failure;
        const bool outer_inplace = plan->placement == rocfft_placement_inplace;
        if(!outer_inplace && !out)
            return rocfft_status_failure;
        const bool multi = gp->comm != nullptr;
        const bool owner = !multi || gp->rank == 0;
        if(owner && !gp->inner)
            return rocfft_status_failure;
        int cur = 0;
        cudaGetDevice(&cur);
        if(cur != gp->device)
            cudaSetDevice(gp->device);
        cudaStream_t s    = info->stream;
        auto         done = [&](rocfft_status v) {
            if(cur != gp->device)
                cudaSetDevice(cur);
            return v;
        };
        // copies between a strided brick (or its packed travel copy) and a box of a contiguous array
        auto to_array = [&](void* array, int elem, const BoxCopy& c, const void* brick) {
            ++g_launch_count;
            return b200fft_launch_brick_copy(static_cast<char*>(array) + c.full_offset * elem, brick, elem, c.n,
                                             c.full_stride, c.brick_stride, s)
                   == cudaSuccess;
        };
        auto from_array = [&](const void* array, int elem, const BoxCopy& c, void* brick) {
            ++g_launch_count;
            return b200fft_launch_brick_copy(brick, static_cast<const char*>(array) + c.full_offset * elem, elem, c.n,
                                             c.brick_stride, c.full_stride, s)
                   == cudaSuccess;
        };
        void* const* dstp = outer_inplace ? in : out;
        for(size_t i = 0; i < gp->gathers.size(); ++i)
            if(!in[i])
                return done(rocfft_status_failure);
        for(size_t j = 0; j < gp->scatters.size(); ++j)
            if(!dstp[j])
                return done(rocfft_status_failure);
        NcclApi& N       = nccl();
        char*    staging = static_cast<char*>(gp->staging);

        if(!owner)
        {
            // pack and send the input bricks, receive and unpack the output bricks
            for(size_t i = 0; i < gp->mine_in.size(); ++i)
                if(!to_array(staging + gp->mine_in[i].staging_off, gp->in_elem, gp->mine_in[i].box, in[i]))
                    return done(rocfft_status_failure);
            bool ok = N.GroupStart() == ncclSuccess;
            for(const auto& r : gp->mine_in)
                ok = ok && N.Send(staging + r.staging_off, r.bytes, ncclChar, 0, gp->comm, s) == ncclSuccess;
            ok = ok && N.GroupEnd() == ncclSuccess;
            ok = ok && N.GroupStart() == ncclSuccess;
            for(const auto& r : gp->mine_out)
                ok = ok && N.Recv(staging + r.staging_off, r.bytes, ncclChar, 0, gp->comm, s) == ncclSuccess;
            ok = ok && N.GroupEnd() == ncclSuccess;
            if(!ok)
                return done(rocfft_status_failure);
            for(size_t j = 0; j < gp->mine_out.size(); ++j)
                if(!from_array(staging + gp->mine_out[j].staging_off, gp->out_elem, gp->mine_out[j].box, dstp[j]))
                    return done(rocfft_status_failure);
            return done(rocfft_status_success);
        }

        for(size_t i = 0; i < gp->gathers.size(); ++i)
            if(!to_array(gp->full_in, gp->in_elem, gp->gathers[i], in[i]))
                return done(rocfft_status_failure);
        if(multi && !gp->remote_in.empty())
        {
            bool ok = N.GroupStart() == ncclSuccess;
            for(const auto& r : gp->remote_in)
                ok = ok && N.Recv(staging + r.staging_off, r.bytes, ncclChar, r.owner, gp->comm, s) == ncclSuccess;
            ok = ok && N.GroupEnd() == ncclSuccess;
            if(!ok)
                return done(rocfft_status_failure);
            for(const auto& r : gp->remote_in)
                if(!to_array(gp->full_in, gp->in_elem, r.box, staging + r.staging_off))
                    return done(rocfft_status_failure);
        }
        {
            rocfft_execution_info_t ei    = *info;
            void*                   ib[1] = {gp->full_in};
            void*                   ob[1] = {gp->full_out};
            const rocfft_status     st    = rocfft_execute(gp->inner, ib, gp->inplace ? nullptr : ob, &ei);
            if(st != rocfft_status_success)
                return done(st);
        }
        for(size_t j = 0; j < gp->scatters.size(); ++j)
            if(!from_array(gp->full_out, gp->out_elem, gp->scatters[j], dstp[j]))
                return done(rocfft_status_failure);
        if(multi && !gp->remote_out.empty())
        {
            for(const auto& r : gp->remote_out)
                if(!from_array(gp->full_out, gp->out_elem, r.box, staging + r.staging_off))
                    return done(rocfft_status_failure);
            bool ok = N.GroupStart() == ncclSuccess;
            for(const auto& r : gp->remote_out)
                ok = ok && N.Send(staging + r.staging_off, r.bytes, ncclChar, r.owner, gp->comm, s) == ncclSuccess;
            ok = ok && N.GroupEnd() == ncclSuccess;
            if(!ok)
                return done(rocfft_status_failure);
        }
        if(gp->remote && cudaStreamSynchronize(s) != cudaSuccess)
            return done(rocfft_status_failure);
        return done(rocfft_status_success);
    }
}
