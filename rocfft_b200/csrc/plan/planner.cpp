// Planner: turns a normalised transform description into a flat list of
// kernel launches.
//
// Role in the reference:
//   scheme decision ....... library/src/node_factory.cpp:539-967
//   plan-tree construction  library/src/tree_node_{1D,2D,3D,real,bluestein}.cpp
//   buffer assignment ..... library/src/assignment_policy.cpp:578-1365
//   work-buffer sizing .... library/src/plan.cpp:4439-4473
//
// Design: an N-dimensional transform is a sequence of batched 1D stages, one
// per dimension.  Every Stockham tile kernel accepts arbitrary element and
// batch strides and is safe in place, so stages after the first run in place
// on the output array and no transposes or intermediate buffers are needed
// for plain multi-dimensional complex transforms.  A stage is realised as
//   - one tile kernel when the length is in the function pool (row tiles when
//     the transform dimension is contiguous, column tiles when another
//     dimension is: the SBCC / SBRC / SBCR modes of the reference),
//   - a two-kernel N = N1*N2 decomposition with a twiddle multiply in between
//     when it is not (reference: CS_L1D_CC, tree_node_1D.cpp:319-673),
//   - Bluestein's algorithm for everything else
//     (reference: tree_node_bluestein.cpp:63-408).
// Real transforms wrap a half-length complex stage in pre/post-processing
// (reference: tree_node_real.cpp:211-449).
#include "planner_impl.h"
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <sstream>
#include <stdexcept>

namespace b200fft
{
    PlanCore::~PlanCore()
    {
        int prev = 0;
        cudaGetDevice(&prev);
        if(prev != device)
            cudaSetDevice(device);
        for(void* p : tables)
            cudaFree(p);
        if(prev != device)
            cudaSetDevice(prev);
    }

    using namespace detail;
    namespace
    {
        bool is_planar(rocfft_array_type t)
        {
            return t == rocfft_array_type_complex_planar || t == rocfft_array_type_hermitian_planar;
        }
    } // namespace

    void build_single_device_plan(rocfft_plan_t* plan)
    {
        if(plan->precision == rocfft_precision_half)
            throw std::runtime_error("half precision is not supported");
        auto core       = std::make_unique<PlanCore>();
        core->precision = plan->precision == rocfft_precision_single ? 0 : 1;
        cudaGetDevice(&core->device);
        const size_t rsize = core->precision == 0 ? 4 : 8;

        const auto& d       = plan->desc;
        const bool  inplace = plan->placement == rocfft_placement_inplace;

        DataView in, out;
        in.len    = plan->lengths;
        out.len   = plan->outputLengths;
        in.batch  = plan->batch;
        out.batch = plan->batch;
        for(size_t k = 0; k < plan->rank; ++k)
        {
            in.stride.push_back((ptrdiff_t)d.inStrides[k]);
            out.stride.push_back((ptrdiff_t)d.outStrides[k]);
        }
        in.dist  = (ptrdiff_t)d.inDist;
        out.dist = (ptrdiff_t)d.outDist;

        auto setbuf = [&](DataView& v, rocfft_array_type t, const size_t* off, BufId id) {
            v.buf.id     = id;
            v.buf.planar = is_planar(t);
            if(t == rocfft_array_type_real)
            {
                v.kind            = EK_REAL;
                v.buf.byte_off[0] = off[0] * rsize;
            }
            else if(v.buf.planar)
            {
                v.kind            = EK_CPLX_PL;
                v.buf.byte_off[0] = off[0] * rsize;
                v.buf.byte_off[1] = off[1] * rsize;
            }
            else
            {
                v.kind            = EK_CPLX_IL;
                v.buf.byte_off[0] = off[0] * 2 * rsize;
            }
        };
        setbuf(in, d.inArrayType, d.inOffset, BUF_USER_IN);
        setbuf(out, d.outArrayType, d.outOffset, inplace ? BUF_USER_IN : BUF_USER_OUT);

        Planner p(*core);
        switch(plan->transformType)
        {
        case rocfft_transform_type_complex_forward:
        case rocfft_transform_type_complex_inverse:
        {
            p.plan_c2c(in,
                       out,
                       plan->transformType == rocfft_transform_type_complex_inverse,
                       d.scale,
                       inplace);
            break;
        }
        case rocfft_transform_type_real_forward:
            p.plan_real_forward(in, out, d.scale);
            break;
        case rocfft_transform_type_real_inverse:
            p.plan_real_inverse(in, out, d.scale);
            break;
        }
        plan->core = std::move(core);
    }

    std::string describe_core(const PlanCore& core)
    {
        std::ostringstream o;
        o << "precision: " << (core.precision == 0 ? "single" : "double") << "\n"
          << "work buffer bytes: " << core.work_bytes << "\n"
          << "steps: " << core.steps.size() << "\n";
        int i = 0;
        for(const Step& s : core.steps)
        {
            o << "  [" << i++ << "] " << s.note;
            auto buf = [](const BufRef& b) {
                const char* names[] = {"in", "out", "temp", "plan"};
                return std::string(names[b.id]) + "+" + std::to_string(b.byte_off[0]);
            };
            o << "  " << buf(s.in) << " -> " << buf(s.out);
            if(s.kind == Step::TILE)
                o << "  tiles=" << s.ntiles << " threads=" << s.kern->threads << " smem=" << s.kern->smem_bytes
                  << " outer=(" << s.ka.on[0] << "," << s.ka.on[1] << "," << s.ka.on[2] << ")"
                  << " es=(" << s.ka.in.es << "," << s.ka.out.es << ")";
            else if(s.kind == Step::EW)
                o << "  n=" << s.ea.n << " outer=(" << s.ea.on[0] << "," << s.ea.on[1] << "," << s.ea.on[2] << ")";
            if(!s.loops.empty())
                o << " hostloops=" << s.loops.size();
            o << "\n";
        }
        return o.str();
    }
} // namespace b200fft
