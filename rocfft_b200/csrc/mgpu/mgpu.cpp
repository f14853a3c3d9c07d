// Multi-device layer: slab-decomposed 3D complex transforms across the ranks of
// an NCCL communicator, one process per GPU.
//
// Role in the reference: library/src/plan.cpp:2222-2358 (BuildOptMultiDevicePlan),
// :1908-2220 (GlobalTranspose: pack -> all-to-all -> unpack) and
// library/src/tree_node.cpp:846-901 (CommAllToAllv over MPI_Ialltoallv).
//
// Design (differs from the reference on purpose):
//   * The exchange crosses NVLink as plain peer stores issued by the FFT kernels themselves
//     (default), or as NCCL grouped send/recv (option); never MPI.
//   * There are no pack or unpack kernels.  The three local FFT passes write
//     and read the exchange buffers in packed order themselves:
//       pass A  FFT along Y (column tiles) of the local Z-slab; its store splits Y
//               into per-destination blocks (two-level stride), so every
//               destination's data is one contiguous block;
//       a2a #1  rank q receives (all z, y in Yq, x): blocks arrive in z order,
//               which makes the receive buffer the contiguous array T[z][y_local][x];
//       pass B  FFT along Z (column tiles) on T, store split into per-destination
//               z blocks;
//       a2a #2  back to Z-slabs;
//       pass C  FFT along X (row kernel) reads the staging blocks through its three
//               outer strides and writes the caller's slab in natural order.
//     Three HBM round trips per rank in total, the minimum for a 3D transform
//     without on-chip plane residency.
//   * Default exchange: none as a separate step.  The receive buffers belong to the
//     plan and are mapped into every rank with CUDA IPC; passes A and B get a table
//     of per-destination base pointers and store each block straight into the owning
//     rank's buffer over NVLink while they compute (plain peer stores: no multimem, no
//     TMA).  A one-word NCCL all-reduce on the caller's stream is the barrier between
//     phases.  The plan then needs no caller work buffer.
//   * Rank-2 transforms on row slabs use the same machinery with one transform less: the
//     first phase is a strided copy of every row's x-ranges into the owning ranks'
//     T[y][x_local], the second the FFT along Y with its store split over the ranks'
//     row buffers (natural order), the third the FFT along X.
//   * ROCFFT_B200_MGPU_NCCL=1 selects NCCL grouped send/recv instead: the work is
//     cut into chunks; chunk c+1 is transformed while chunk c is on the wire (compute
//     on the caller's stream, NCCL on an internal stream, events in between).
#include "mgpu.h"
#include "../plan/planner_impl.h"
#include <cstdio>
#include <cstdlib>
#include <dlfcn.h>
#include <mutex>
#include <nccl.h>

namespace b200fft
{
    NcclApi& nccl()
        {
            static NcclApi        api;
            static std::once_flag once;
            std::call_once(once, [] {
                for(const char* name : {"libnccl.so.2", "libnccl.so"})
                {
                    api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
                    if(api.handle)
                        break;
                }
                if(!api.handle)
                    return;
                auto sym = [&](const char* n) { return dlsym(api.handle, n); };
                api.GetUniqueId    = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
                api.CommInitRank   = (decltype(api.CommInitRank))sym("ncclCommInitRank");
                api.CommDestroy    = (decltype(api.CommDestroy))sym("ncclCommDestroy");
                api.CommCount      = (decltype(api.CommCount))sym("ncclCommCount");
                api.CommUserRank   = (decltype(api.CommUserRank))sym("ncclCommUserRank");
                api.Send           = (decltype(api.Send))sym("ncclSend");
                api.Recv           = (decltype(api.Recv))sym("ncclRecv");
                api.GroupStart     = (decltype(api.GroupStart))sym("ncclGroupStart");
                api.GroupEnd       = (decltype(api.GroupEnd))sym("ncclGroupEnd");
                api.AllGather      = (decltype(api.AllGather))sym("ncclAllGather");
                api.AllReduce      = (decltype(api.AllReduce))sym("ncclAllReduce");
                api.GetErrorString = (decltype(api.GetErrorString))sym("ncclGetErrorString");
                api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.CommCount && api.CommUserRank
                         && api.Send && api.Recv && api.GroupStart && api.GroupEnd && api.AllGather && api.AllReduce;
            });
            return api;
        }

    namespace
    {
        void nccl_check(ncclResult_t r, const char* what)
        {
            if(r != ncclSuccess)
            {
                std::string msg = std::string(what) + ": ";
                msg += nccl().GetErrorString ? nccl().GetErrorString(r) : "NCCL error";
                throw std::runtime_error(msg);
            }
        }

        struct SlabPlan
        {
            MultiDeviceHeader hdr{0};
            ncclComm_t comm  = nullptr;
            int        P     = 1;
            int        rank  = 0;
            size_t     csize = 8;
            size_t     nx = 1, ny = 1, nz = 1;
            size_t     nb = 1; // transforms per plan (batch); every rank holds its slab of each
            size_t     lz = 1, ly = 1; // local extents: nz / P, ny / P
            int        chunks = 1;
            size_t     slab_bytes = 0;
            size_t     off_s = 0, off_r = 0, off_r2 = 0; // work-buffer layout
            size_t     work_bytes = 0;
            std::vector<std::unique_ptr<PlanCore>> passA, passB, passC; // one per chunk
            cudaStream_t             comm_stream = nullptr;
            std::vector<cudaEvent_t> evA, evB, evX;
            cudaEvent_t              ev_all = nullptr, ev_start = nullptr;
            int                      device  = 0;
            // peer-to-peer mode: the FFT passes store straight into the other ranks' receive
            // buffers (plan-owned, shared through CUDA IPC); NCCL only provides the barriers
            bool               p2p = false;
            void *             R = nullptr, *R2 = nullptr; // this rank's receive buffers
            std::vector<void*> peer_r, peer_r2; // every rank's buffers as mapped here
            void **            tab_a = nullptr, **tab_b = nullptr; // device tables of block bases
            int*               bar   = nullptr; // device words for the barrier all-reduce
            // Output split along X instead of Z (the reference's "slow in, fast out" layout): one global
            // transpose instead of two.  passA = X rows into the plan-owned array S, passB = Y columns stored
            // straight into the peers' R (one launch per destination), passC = Z columns from R to the caller.
            bool  xsplit = false;
            void* S      = nullptr;
            // Rank-2 transforms on row slabs (rank q holds rows y in [q*ly, (q+1)*ly) of every image, in and
            // out): passA = the rows' x-ranges copied straight into the owning ranks' R, which then hold
            // T[y][x_local]; passB = Y columns of T, stored into the peers' R2 in the natural order
            // [y_local][x]; passC = X rows from R2 to the caller.
            bool rows2d = false;
        };

        size_t total_work(const SlabPlan& sp)
        {
            size_t w = sp.work_bytes;
            for(auto* v : {&sp.passA, &sp.passB, &sp.passC})
                for(auto& c : *v)
                    w = std::max(w, c->work_bytes);
            return w;
        }
    }

    // Byte offsets of the blocks one rank sends and receives in one chunk of one
    // exchange.  Offsets are relative to the send buffer S and to the receive
    // buffer (R for the first exchange, the staging buffer R2 for the second).
    //   first exchange : block for rank q starts at S + c*chunk + q*blk; the block
    //                    from rank q lands at R + (q*chunks + c)*blk, which places
    //                    its planes at z = q*lz + c*cz of T[z][y_local][x];
    //   second exchange: send as above; the block from rank q lands at
    //                    R2 + c*chunk + q*blk, i.e. R2_c[q][z_local][yc][x].
    void slab_exchange_offsets(int     ranks,
                               int     chunks,
                               size_t  slab_bytes,
                               int     first,
                               int     c,
                               size_t* send_off,
                               size_t* recv_off,
                               size_t* block_bytes)
    {
        const size_t chunk_bytes = slab_bytes / (size_t)chunks;
        const size_t blk         = chunk_bytes / (size_t)ranks;
        *block_bytes             = blk;
        for(int q = 0; q < ranks; ++q)
        {
            send_off[q] = (size_t)c * chunk_bytes + (size_t)q * blk;
            recv_off[q] = first ? ((size_t)q * chunks + c) * blk : (size_t)c * chunk_bytes + (size_t)q * blk;
        }
    }

    void rows2d_exchange_offsets(int ranks, int rank, size_t nx, size_t ny, size_t elem_bytes, size_t* first_off, size_t* second_off)
    {
        const size_t lx = nx / (size_t)ranks, ly = ny / (size_t)ranks;
        *first_off      = (size_t)rank * ly * lx * elem_bytes; // rows y = rank*ly ... of T[y][x_local]
        *second_off     = (size_t)rank * lx * elem_bytes; // columns x = rank*lx ... of every row of [y_local][x]
    }

    void build_multi_device_plan(rocfft_plan_t* plan)
    {
        const auto& d = plan->desc;
        if(d.inFields.size() != 1 || d.outFields.size() != 1)
            throw std::runtime_error("exactly one input field and one output field are supported");
        if(d.comm_type == rocfft_comm_none)
        {
            // one process drives every brick: gather, transform on one device, scatter
            build_gather_scatter_plan(plan);
            return;
        }
        if(d.comm_type != rocfft_comm_nccl || !d.comm_handle)
            throw std::runtime_error("multi-process plans need an NCCL communicator (rocfft_comm_nccl)");
        if(plan->precision == rocfft_precision_half)
            throw std::runtime_error("half precision is not supported");
        NcclApi& N = nccl();
        if(!N.ok)
            throw std::runtime_error("libnccl could not be loaded");

        auto sp   = std::make_unique<SlabPlan>();
        sp->comm  = *static_cast<ncclComm_t*>(d.comm_handle);
        nccl_check(N.CommCount(sp->comm, &sp->P), "ncclCommCount");
        nccl_check(N.CommUserRank(sp->comm, &sp->rank), "ncclCommUserRank");
        cudaGetDevice(&sp->device);
        sp->csize = plan->precision == rocfft_precision_single ? 8 : 16;
        const int P = sp->P;

        // The optimised plan takes rank-3 complex transforms (any batch) whose fields are one contiguous
        // Z-slab per rank — the slabs of the batch members back to back — in rank order, with lengths
        // divisible by the number of ranks.  Everything else goes through the gather / scatter plan; all
        // ranks must take the same branch, so they agree on it first.
        const bool c2c = plan->transformType == rocfft_transform_type_complex_forward
                         || plan->transformType == rocfft_transform_type_complex_inverse;
        const bool il_c2c = c2c && d.inArrayType == rocfft_array_type_complex_interleaved
                            && d.outArrayType == rocfft_array_type_complex_interleaved && plan->batch >= 1
                            && plan->lengths == plan->userLengths;
        bool slab_ok = il_c2c && plan->rank == 3;
        // rank 2: row slabs in and out, peer-store exchange only, column length one kernel can take
        bool rows_ok = il_c2c && plan->rank == 2 && !getenv("ROCFFT_B200_MGPU_NCCL") && !getenv("ROCFFT_B200_MGPU_NO_ROWS2D");
        if(rows_ok)
        {
            sp->nx = plan->lengths[0];
            sp->ny = plan->lengths[1];
            sp->nz = 1;
            sp->nb = plan->batch;
            const int prec2 = plan->precision == rocfft_precision_single ? 0 : 1;
            rows_ok = sp->ny % P == 0 && sp->nx % P == 0 && detail::pool_find(sp->ny, prec2, B200FFT_COL_BLK) != nullptr;
        }
        if(rows_ok)
        {
            sp->ly = sp->ny / P;
            sp->lz = 1;
            auto is_rows = [&](const rocfft_field_t& f) {
                if(f.bricks.size() != 1)
                    return false;
                const rocfft_brick_t& b = f.bricks[0];
                if(b.lower.size() != 3 || b.upper.size() != 3 || b.stride.size() != 3)
                    return false;
                const size_t lo[3] = {0, sp->rank * sp->ly, 0};
                const size_t hi[3] = {sp->nx, (sp->rank + 1) * sp->ly, sp->nb};
                const size_t st[3] = {1, sp->nx, sp->nx * sp->ly};
                for(int i = 0; i < 3; ++i)
                    if(b.lower[i] != lo[i] || b.upper[i] != hi[i] || ((i < 2 || sp->nb > 1) && b.stride[i] != st[i]))
                        return false;
                return true;
            };
            rows_ok = is_rows(d.inFields[0]) && is_rows(d.outFields[0]);
        }
        // the NCCL send/recv exchange moves one transform's slab; batches use the peer-store exchange
        if(plan->batch > 1 && getenv("ROCFFT_B200_MGPU_NCCL"))
            slab_ok = false;
        if(slab_ok)
        {
            sp->nx  = plan->lengths[0];
            sp->ny  = plan->lengths[1];
            sp->nz  = plan->lengths[2];
            sp->nb  = plan->batch;
            slab_ok = sp->nz % P == 0 && sp->ny % P == 0;
        }
        if(slab_ok)
        {
            sp->lz = sp->nz / P;
            sp->ly = sp->ny / P;
            auto is_slab = [&](const rocfft_field_t& f) {
                if(f.bricks.size() != 1)
                    return false;
                const rocfft_brick_t& b = f.bricks[0];
                if(b.lower.size() != 4 || b.upper.size() != 4 || b.stride.size() != 4)
                    return false;
                const size_t lo[4] = {0, 0, sp->rank * sp->lz, 0};
                const size_t hi[4] = {sp->nx, sp->ny, (sp->rank + 1) * sp->lz, sp->nb};
                const size_t st[4] = {1, sp->nx, sp->nx * sp->ny, sp->nx * sp->ny * sp->lz};
                for(int i = 0; i < 4; ++i)
                    if(b.lower[i] != lo[i] || b.upper[i] != hi[i] || ((i < 3 || sp->nb > 1) && b.stride[i] != st[i]))
                        return false;
                return true;
            };
            const bool in_slab = is_slab(d.inFields[0]);
            // output split along the fastest dimension: rank q holds x in [q*lx, (q+1)*lx) of every row
            auto is_xsplit = [&](const rocfft_field_t& f) {
                if(f.bricks.size() != 1 || sp->nx % P != 0 || getenv("ROCFFT_B200_MGPU_NCCL"))
                    return false;
                const rocfft_brick_t& b = f.bricks[0];
                if(b.lower.size() != 4 || b.upper.size() != 4 || b.stride.size() != 4)
                    return false;
                const size_t lx    = sp->nx / P;
                const size_t lo[4] = {sp->rank * lx, 0, 0, 0};
                const size_t hi[4] = {(sp->rank + 1) * lx, sp->ny, sp->nz, sp->nb};
                const size_t st[4] = {1, lx, lx * sp->ny, lx * sp->ny * sp->nz};
                for(int i = 0; i < 4; ++i)
                    if(b.lower[i] != lo[i] || b.upper[i] != hi[i] || ((i < 3 || sp->nb > 1) && b.stride[i] != st[i]))
                        return false;
                return true;
            };
            // (with a single rank both descriptions fit; the two-transpose plan is kept unless a test asks otherwise)
            const bool out_slab = is_slab(d.outFields[0]);
            sp->xsplit = in_slab && is_xsplit(d.outFields[0]) && (!out_slab || getenv("ROCFFT_B200_MGPU_PREFER_XSPLIT"));
            slab_ok    = in_slab && (sp->xsplit || out_slab);
        }
        {
            // 0: not a slab layout, 1: slabs in and out, 2: slabs in, X-split out, 3: row slabs of a rank-2
            // transform; every rank must say the same
            if(rows_ok)
                slab_ok = true;
            sp->rows2d = rows_ok;
            int  mine = slab_ok ? (rows_ok ? 3 : (sp->xsplit ? 2 : 1)) : 0;
            int* dbuf = nullptr;
            if(cudaMalloc(&dbuf, sizeof(int) * (P + 1)) != cudaSuccess)
                throw std::runtime_error("cudaMalloc failed");
            cudaMemcpy(dbuf, &mine, sizeof mine, cudaMemcpyHostToDevice);
            ncclResult_t     r = N.AllGather(dbuf, dbuf + 1, sizeof mine, ncclChar, sp->comm, nullptr);
            cudaError_t      e = cudaStreamSynchronize(nullptr);
            std::vector<int> all(P);
            cudaMemcpy(all.data(), dbuf + 1, sizeof(int) * P, cudaMemcpyDeviceToHost);
            cudaFree(dbuf);
            nccl_check(r, "ncclAllGather");
            if(e != cudaSuccess)
                throw std::runtime_error("brick exchange failed");
            for(int v : all)
                slab_ok = slab_ok && v == mine && v != 0;
        }
        if(!slab_ok && !getenv("ROCFFT_B200_MGPU_NO_GATHER"))
        {
            build_gather_scatter_plan(plan);
            return;
        }
        if(!slab_ok)
            throw std::runtime_error("brick layout is not one Z-slab per rank");

        // Exchange mode.  Default: peer-to-peer stores from inside the FFT kernels.
        // ROCFFT_B200_MGPU_NCCL=1 selects the NCCL send/recv exchange instead.
        sp->p2p = getenv("ROCFFT_B200_MGPU_NCCL") == nullptr;

        // Chunking (NCCL mode only): every pass is cut into k chunks so that chunk c+1 computes while chunk c is
        // on the wire.  The peer-store mode runs whole passes: cutting passes B and C into chunks and running the
        // row pass C of chunk c on a second stream beside pass B of chunk c+1 was measured on two GPUs (1024^3)
        // and gained nothing — B + C took 4.48 ms overlapped against 3.03 + 1.32 ms in sequence: pass B keeps
        // the SMs busy although its stores cross NVLink — so that variant was dropped.
        int k = 4;
        if(const char* env = getenv("ROCFFT_B200_MGPU_CHUNKS"))
            k = std::max(1, atoi(env));
        while(k > 1 && (sp->lz % k || sp->ly % k))
            k /= 2;
        if(sp->p2p)
            k = 1;
        sp->chunks = k;
        const int kA = k; // chunks of pass A

        const size_t nx = sp->nx, ny = sp->ny, lz = sp->lz, ly = sp->ly;
        const size_t cz = lz / kA, cy = ly / k;
        const size_t slab_elems = sp->rows2d ? nx * ly : nx * ny * lz; // one batch member's slab
        const size_t nb         = sp->nb;
        sp->slab_bytes          = slab_elems * sp->csize;
        const int  prec         = plan->precision == rocfft_precision_single ? 0 : 1;
        const bool inverse      = plan->transformType == rocfft_transform_type_complex_inverse;
        const bool inplace      = plan->placement == rocfft_placement_inplace;

        using namespace detail;
        auto new_core = [&]() {
            auto c       = std::make_unique<PlanCore>();
            c->precision = prec;
            c->device    = sp->device;
            return c;
        };
        // work buffer: S | R | R2, then whatever scratch the passes ask for (none today)
        auto align = [](size_t v) { return (v + 255) & ~size_t(255); };
        sp->off_s  = 0;
        sp->off_r  = align(sp->slab_bytes * nb);
        sp->off_r2 = sp->off_r + align(sp->slab_bytes * nb);
        sp->work_bytes = sp->off_r2 + align(sp->slab_bytes * nb);

        BufRef user_in, user_out, S, R, R2;
        user_in.id  = BUF_USER_IN;
        user_out.id = inplace ? BUF_USER_IN : BUF_USER_OUT;
        S.id = R.id = R2.id = BUF_TEMP;
        const size_t chunk_bytes = sp->slab_bytes / k;

        if(sp->p2p)
        {
            // Plan-owned receive buffers, visible to every rank through CUDA IPC.
            int ndev = 0;
            if(cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
                sp->p2p = false; // no GPU in this process: the plan stays inspectable only
        }
        if((sp->xsplit || sp->rows2d) && !sp->p2p)
            throw std::runtime_error("this plan needs a GPU and the peer-store exchange");
        if(sp->xsplit && cudaMalloc(&sp->S, sp->slab_bytes * nb) != cudaSuccess)
            throw std::runtime_error("intermediate array allocation failed");
        if(sp->p2p)
        {
            if(cudaMalloc(&sp->R, sp->slab_bytes * nb) != cudaSuccess || cudaMalloc(&sp->R2, sp->slab_bytes * nb) != cudaSuccess)
                throw std::runtime_error("exchange buffer allocation failed");
            sp->peer_r.assign(P, nullptr);
            sp->peer_r2.assign(P, nullptr);
            if(P == 1)
            {
                sp->peer_r[0]  = sp->R;
                sp->peer_r2[0] = sp->R2;
            }
            else
            {
                cudaIpcMemHandle_t mine[2];
                if(cudaIpcGetMemHandle(&mine[0], sp->R) != cudaSuccess
                   || cudaIpcGetMemHandle(&mine[1], sp->R2) != cudaSuccess)
                    throw std::runtime_error("cudaIpcGetMemHandle failed");
                char* dbuf = nullptr;
                if(cudaMalloc(&dbuf, sizeof(mine) * (P + 1)) != cudaSuccess)
                    throw std::runtime_error("cudaMalloc failed");
                cudaMemcpy(dbuf, mine, sizeof mine, cudaMemcpyHostToDevice);
                ncclResult_t r = N.AllGather(dbuf, dbuf + sizeof(mine), sizeof mine, ncclChar, sp->comm, nullptr);
                cudaError_t  e = cudaStreamSynchronize(nullptr);
                std::vector<cudaIpcMemHandle_t> all(2 * P);
                cudaMemcpy(all.data(), dbuf + sizeof(mine), sizeof(mine) * P, cudaMemcpyDeviceToHost);
                cudaFree(dbuf);
                nccl_check(r, "ncclAllGather");
                if(e != cudaSuccess)
                    throw std::runtime_error("IPC handle exchange failed");
                for(int q = 0; q < P; ++q)
                {
                    if(q == sp->rank)
                    {
                        sp->peer_r[q]  = sp->R;
                        sp->peer_r2[q] = sp->R2;
                        continue;
                    }
                    if(cudaIpcOpenMemHandle(&sp->peer_r[q], all[2 * q], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess
                       || cudaIpcOpenMemHandle(&sp->peer_r2[q], all[2 * q + 1], cudaIpcMemLazyEnablePeerAccess)
                              != cudaSuccess)
                        throw std::runtime_error("cudaIpcOpenMemHandle failed (peer access between the GPUs is required)");
                }
            }
            // block q of pass A lands in rank q's T at planes z = rank*lz ..., block q of pass B in
            // rank q's staging buffer at part `rank`; both are rank * (slab / P) bytes into the buffer
            // (pass B chunk c: the staging buffer holds chunk after chunk, and inside a chunk one part per source rank)
            const size_t       part = sp->slab_bytes / P;
            std::vector<void*> ta(P), tb((size_t)P * k);
            for(int q = 0; q < P; ++q)
            {
                ta[q] = static_cast<char*>(sp->peer_r[q]) + (size_t)sp->rank * part;
                for(int c = 0; c < k; ++c)
                    tb[(size_t)c * P + q] = static_cast<char*>(sp->peer_r2[q]) + (size_t)c * (sp->slab_bytes / k)
                                            + (size_t)sp->rank * (part / k);
                // row slabs: this rank's columns x in [rank*lx, (rank+1)*lx) of every row of rank q's [y_local][x]
                if(sp->rows2d)
                {
                    size_t o1 = 0, o2 = 0;
                    rows2d_exchange_offsets(P, sp->rank, sp->nx, sp->ny, sp->csize, &o1, &o2);
                    tb[q] = static_cast<char*>(sp->peer_r2[q]) + o2;
                }
            }
            if(cudaMalloc(&sp->tab_a, sizeof(void*) * P) != cudaSuccess
               || cudaMalloc(&sp->tab_b, sizeof(void*) * P * k) != cudaSuccess || cudaMalloc(&sp->bar, 64) != cudaSuccess)
                throw std::runtime_error("cudaMalloc failed");
            cudaMemcpy(sp->tab_a, ta.data(), sizeof(void*) * P, cudaMemcpyHostToDevice);
            cudaMemcpy(sp->tab_b, tb.data(), sizeof(void*) * P * k, cudaMemcpyHostToDevice);
            cudaMemset(sp->bar, 0, 64);
            S.id = R.id = R2.id = BUF_ABS;
            sp->off_s  = 0;
            sp->off_r  = reinterpret_cast<size_t>(sp->R);
            sp->off_r2 = reinterpret_cast<size_t>(sp->R2);
            sp->work_bytes = 0;
        }

        if(sp->rows2d)
        {
            const size_t lx = nx / P;
            BufRef       Rb, R2b;
            Rb.id = R2b.id  = BUF_ABS;
            Rb.byte_off[0]  = reinterpret_cast<size_t>(sp->R);
            R2b.byte_off[0] = reinterpret_cast<size_t>(sp->R2);
            // pass A: no arithmetic.  The x-range of rank q goes from the caller's rows into rank q's
            // R = T[b][y][x_local] at rows y = rank*ly ...: one strided copy per destination, plain peer stores
            {
                auto    core = new_core();
                Planner p(*core);
                for(int q = 0; q < P; ++q)
                {
                    Stage s;
                    s.n  = 1;
                    s.is = s.os = 1;
                    s.outer.push_back({lx, 1, 1});
                    s.outer.push_back({ly, (ptrdiff_t)nx, (ptrdiff_t)lx});
                    s.outer.push_back({nb, (ptrdiff_t)slab_elems, (ptrdiff_t)(ny * lx)});
                    s.in              = user_in;
                    s.in.byte_off[0]  = (size_t)q * lx * sp->csize;
                    s.out             = Rb;
                    size_t o1 = 0, o2 = 0;
                    rows2d_exchange_offsets(P, sp->rank, nx, ny, sp->csize, &o1, &o2);
                    s.out.byte_off[0] = reinterpret_cast<size_t>(sp->peer_r[q]) + o1;
                    p.emit_c2c_1d(s);
                }
                sp->passA.push_back(std::move(core));
            }
            // pass B: FFT along Y on T; output point y belongs to rank y / ly, whose R2 is laid out like the
            // caller's slab, [b][y_local][x]: the store splits Y into per-destination blocks
            {
                auto    core = new_core();
                Planner p(*core);
                Stage   s;
                s.n       = ny;
                s.is      = (ptrdiff_t)lx;
                s.os      = (ptrdiff_t)nx;
                s.out_blk = ly;
                s.out_bs  = 0;
                s.outer.push_back({lx, 1, 1});
                s.outer.push_back({nb, (ptrdiff_t)(ny * lx), (ptrdiff_t)slab_elems});
                s.in           = Rb;
                s.out          = R2b;
                s.out_blk_ptrs = sp->tab_b;
                s.peer_out     = P > 1;
                s.inverse      = inverse;
                p.emit_c2c_1d(s);
                sp->passB.push_back(std::move(core));
            }
            // pass C: FFT along X, R2 -> the caller's slab
            {
                auto    core = new_core();
                Planner p(*core);
                Stage   s;
                s.n  = nx;
                s.is = s.os = 1;
                s.outer.push_back({ly, (ptrdiff_t)nx, (ptrdiff_t)nx});
                s.outer.push_back({nb, (ptrdiff_t)slab_elems, (ptrdiff_t)slab_elems});
                s.in      = R2b;
                s.out     = user_out;
                s.inverse = inverse;
                if(d.scale != 1.0)
                {
                    s.use_scale = true;
                    s.scale     = d.scale;
                }
                p.emit_c2c_1d(s);
                sp->passC.push_back(std::move(core));
            }
        }
        else if(sp->xsplit)
        {
            const size_t lx = nx / P;
            BufRef       Sb, Rb;
            Sb.id = Rb.id  = BUF_ABS;
            Sb.byte_off[0] = reinterpret_cast<size_t>(sp->S);
            Rb.byte_off[0] = reinterpret_cast<size_t>(sp->R);
            // pass A: FFT along X (rows) of the local slab(s): caller's input -> S, same layout
            {
                auto    core = new_core();
                Planner p(*core);
                Stage   s;
                s.n  = nx;
                s.is = s.os = 1;
                s.outer.push_back({ny, (ptrdiff_t)nx, (ptrdiff_t)nx});
                s.outer.push_back({lz, (ptrdiff_t)(nx * ny), (ptrdiff_t)(nx * ny)});
                s.outer.push_back({nb, (ptrdiff_t)slab_elems, (ptrdiff_t)slab_elems});
                s.in      = user_in;
                s.out     = Sb;
                s.inverse = inverse;
                p.emit_c2c_1d(s);
                sp->passA.push_back(std::move(core));
            }
            // pass B: FFT along Y; the columns x in [q*lx, (q+1)*lx) go to rank q, which receives
            // R[b][z][y][x_local] with z = rank*lz + z_local: one launch per destination, plain peer stores
            {
                auto    core = new_core();
                Planner p(*core);
                for(int q = 0; q < P; ++q)
                {
                    Stage s;
                    s.n  = ny;
                    s.is = (ptrdiff_t)nx;
                    s.os = (ptrdiff_t)lx;
                    s.outer.push_back({lx, 1, 1});
                    s.outer.push_back({lz, (ptrdiff_t)(nx * ny), (ptrdiff_t)(ny * lx)});
                    s.outer.push_back({nb, (ptrdiff_t)slab_elems, (ptrdiff_t)(sp->nz * ny * lx)});
                    s.in             = Sb;
                    s.in.byte_off[0] = reinterpret_cast<size_t>(sp->S) + (size_t)q * lx * sp->csize;
                    s.out            = Rb;
                    s.out.byte_off[0]
                        = reinterpret_cast<size_t>(sp->peer_r[q]) + (size_t)sp->rank * lz * ny * lx * sp->csize;
                    s.peer_out = q != sp->rank;
                    s.inverse = inverse;
                    p.emit_c2c_1d(s);
                }
                sp->passB.push_back(std::move(core));
            }
            // pass C: FFT along Z on R[b][z][y][x_local] -> the caller's X-split brick (same index order)
            {
                auto    core = new_core();
                Planner p(*core);
                Stage   s;
                s.n  = sp->nz;
                s.is = (ptrdiff_t)(ny * lx);
                s.os = (ptrdiff_t)(ny * lx);
                s.outer.push_back({ny * lx, 1, 1});
                s.outer.push_back({nb, (ptrdiff_t)(sp->nz * ny * lx), (ptrdiff_t)(sp->nz * ny * lx)});
                s.in      = Rb;
                s.out     = user_out;
                s.inverse = inverse;
                if(d.scale != 1.0)
                {
                    s.use_scale = true;
                    s.scale     = d.scale;
                }
                p.emit_c2c_1d(s);
                sp->passC.push_back(std::move(core));
            }
        }
        else
        for(int c = 0; c < k; ++c)
        {
            // ---- pass A: FFT along Y for z-chunk c, slab -> S_c[q][zc][yq][x]
            if(c < kA)
            {
                auto    core = new_core();
                Planner p(*core);
                Stage   s;
                s.n  = ny;
                s.is = (ptrdiff_t)nx;
                s.os = (ptrdiff_t)nx;
                s.out_blk = ly;
                s.out_bs  = (ptrdiff_t)(cz * ly * nx);
                s.outer.push_back({nx, 1, 1});
                s.outer.push_back({cz, (ptrdiff_t)(nx * ny), (ptrdiff_t)(ly * nx)});
                // batch members: slab after slab on the input side, T after T (nz * ly * nx points each) in the receive buffers
                s.outer.push_back({nb, (ptrdiff_t)slab_elems, (ptrdiff_t)slab_elems});
                s.in             = user_in;
                s.in.byte_off[0] = c * cz * nx * ny * sp->csize;
                s.out            = S;
                s.out.byte_off[0] = sp->off_s + c * (sp->slab_bytes / kA);
                if(sp->p2p)
                    s.out_blk_ptrs = sp->tab_a;
                s.peer_out = sp->p2p && P > 1;
                s.inverse        = inverse;
                p.emit_c2c_1d(s);
                sp->passA.push_back(std::move(core));
            }
            // ---- pass B: FFT along Z for y-chunk c, T[z][y_local][x] -> S2_c[q][zq][yc][x]
            {
                auto    core = new_core();
                Planner p(*core);
                Stage   s;
                s.n  = sp->nz;
                s.is = (ptrdiff_t)(ly * nx);
                s.os = (ptrdiff_t)(cy * nx);
                s.out_blk = lz;
                s.out_bs  = (ptrdiff_t)(lz * cy * nx);
                s.outer.push_back({nx, 1, 1});
                s.outer.push_back({cy, (ptrdiff_t)nx, (ptrdiff_t)nx});
                s.outer.push_back({nb, (ptrdiff_t)slab_elems, (ptrdiff_t)slab_elems});
                s.in              = R;
                s.in.byte_off[0]  = sp->off_r + c * cy * nx * sp->csize;
                s.out             = S;
                s.out.byte_off[0] = sp->off_s + c * chunk_bytes;
                if(sp->p2p)
                    s.out_blk_ptrs = sp->tab_b + (size_t)c * P;
                s.peer_out = sp->p2p && P > 1;
                s.inverse         = inverse;
                p.emit_c2c_1d(s);
                sp->passB.push_back(std::move(core));
            }
            // ---- pass C: FFT along X for y-chunk c, R2_c[r][z_local][yc][x] -> slab
            {
                auto    core = new_core();
                Planner p(*core);
                Stage   s;
                s.n  = nx;
                s.is = s.os = 1;
                s.outer.push_back({cy, (ptrdiff_t)nx, (ptrdiff_t)nx});
                s.outer.push_back({(size_t)P, (ptrdiff_t)(lz * cy * nx), (ptrdiff_t)(ly * nx)});
                s.outer.push_back({lz, (ptrdiff_t)(cy * nx), (ptrdiff_t)(nx * ny)});
                s.outer.push_back({nb, (ptrdiff_t)slab_elems, (ptrdiff_t)slab_elems});
                s.in              = R2;
                s.in.byte_off[0]  = sp->off_r2 + c * chunk_bytes;
                s.out             = user_out;
                s.out.byte_off[0] = c * cy * nx * sp->csize;
                s.inverse         = inverse;
                if(d.scale != 1.0)
                {
                    s.use_scale = true;
                    s.scale     = d.scale;
                }
                p.emit_c2c_1d(s);
                sp->passC.push_back(std::move(core));
            }
        }
        if(!sp->p2p)
            sp->work_bytes = std::max(sp->work_bytes, total_work(*sp));

        bool host_only = false;
        for(auto* v : {&sp->passA, &sp->passB, &sp->passC})
            for(auto& c : *v)
                host_only = host_only || c->host_only;
        if(!host_only)
        {
            cudaStreamCreateWithFlags(&sp->comm_stream, cudaStreamNonBlocking);
            auto mk = [](cudaEvent_t& e) { cudaEventCreateWithFlags(&e, cudaEventDisableTiming); };
            sp->evA.resize(k);
            sp->evB.resize(k);
            sp->evX.resize(k);
            for(int c = 0; c < k; ++c)
            {
                mk(sp->evA[c]);
                mk(sp->evB[c]);
                mk(sp->evX[c]);
            }
            mk(sp->ev_all);
            mk(sp->ev_start);
        }
        plan->mgpu = sp.release();
    }

    void destroy_multi_device_plan(rocfft_plan_t* plan)
    {
        if(multi_device_kind(plan) == 1)
            return destroy_gather_scatter_plan(plan);
        auto* sp = static_cast<SlabPlan*>(plan->mgpu);
        if(!sp)
            return;
        for(auto* v : {&sp->evA, &sp->evB, &sp->evX})
            for(cudaEvent_t e : *v)
                cudaEventDestroy(e);
        if(sp->ev_all)
            cudaEventDestroy(sp->ev_all);
        if(sp->ev_start)
            cudaEventDestroy(sp->ev_start);
        if(sp->comm_stream)
            cudaStreamDestroy(sp->comm_stream);
        if(sp->p2p)
        {
            // Destruction is collective: every rank first unmaps the peers' buffers, then all ranks
            // meet in a barrier, and only then does each free the memory it exported (freeing
            // exported memory while another process still has it mapped is undefined).
            cudaDeviceSynchronize();
            for(int q = 0; q < (int)sp->peer_r.size(); ++q)
            {
                if(q == sp->rank)
                    continue;
                if(sp->peer_r[q])
                    cudaIpcCloseMemHandle(sp->peer_r[q]);
                if(sp->peer_r2[q])
                    cudaIpcCloseMemHandle(sp->peer_r2[q]);
            }
            if(sp->P > 1 && sp->bar && nccl().ok && !getenv("ROCFFT_B200_MGPU_LOCAL_DESTROY"))
            {
                cudaMemsetAsync(sp->bar + 2, 0, sizeof(int), nullptr);
                if(nccl().AllReduce(sp->bar + 2, sp->bar + 10, 1, ncclInt, ncclSum, sp->comm, nullptr) == ncclSuccess)
                    cudaStreamSynchronize(nullptr);
            }
            cudaFree(sp->S);
            cudaFree(sp->tab_a);
            cudaFree(sp->tab_b);
            cudaFree(sp->bar);
            cudaFree(sp->R);
            cudaFree(sp->R2);
        }
        delete sp;
        plan->mgpu = nullptr;
    }

    size_t multi_device_work_bytes(const rocfft_plan_t* plan)
    {
        if(multi_device_kind(plan) == 1)
            return gather_scatter_work_bytes(plan);
        auto* sp = static_cast<const SlabPlan*>(plan->mgpu);
        return sp ? sp->work_bytes : 0;
    }

    std::string describe_multi_device_plan(const rocfft_plan_t* plan)
    {
        if(multi_device_kind(plan) == 1)
            return describe_gather_scatter_plan(plan);
        auto* sp = static_cast<const SlabPlan*>(plan->mgpu);
        if(!sp)
            return "";
        std::ostringstream o;
        o << "slab plan: ranks " << sp->P << " rank " << sp->rank << " lengths " << sp->nx << "x" << sp->ny << "x"
          << sp->nz << " batch " << sp->nb << (sp->xsplit ? " output split along x (one global transpose)" : "")
          << (sp->rows2d ? " row slabs of a rank-2 transform" : "")
          << " chunks " << sp->chunks << " work bytes " << sp->work_bytes << "\n";
        for(int c = 0; c < sp->chunks; ++c)
        {
            o << "chunk " << c << (sp->rows2d ? " pass A (copy):\n" : sp->xsplit ? " pass A (X):\n" : " pass A (Y):\n")
              << describe_core(*sp->passA[c]);
            o << "chunk " << c << (sp->rows2d || sp->xsplit ? " pass B (Y):\n" : " pass B (Z):\n") << describe_core(*sp->passB[c]);
            o << "chunk " << c << (sp->xsplit ? " pass C (Z):\n" : " pass C (X):\n") << describe_core(*sp->passC[c]);
        }
        return o.str();
    }

    std::string multi_device_plan_graph(const rocfft_plan_t* plan)
    {
        std::ostringstream o;
        o << "digraph plan {\n  rankdir=TB;\n";
        if(multi_device_kind(plan) == 1)
        {
            // gather -> one single-device transform -> scatter; the text description names the copies
            o << "  gather [label=\"copy input bricks to one device\"];\n  fft [label=\"single-device transform\"];\n"
                 "  scatter [label=\"copy result to output bricks\"];\n  gather -> fft -> scatter;\n}";
            return o.str();
        }
        auto* sp = static_cast<const SlabPlan*>(plan->mgpu);
        if(!sp)
            return "digraph plan {}";
        auto items = [&](const char* tag, const char* what, const std::vector<std::unique_ptr<PlanCore>>& v) {
            std::vector<std::string> ids;
            for(size_t c = 0; c < v.size(); ++c)
                for(size_t i = 0; i < v[c]->steps.size(); ++i)
                {
                    std::string id = std::string(tag) + std::to_string(c) + "_" + std::to_string(i);
                    o << "  " << id << " [label=\"rank " << sp->rank << ": " << what << " (" << v[c]->steps[i].note << ")\"];\n";
                    ids.push_back(id);
                }
            return ids;
        };
        const char* wa = sp->rows2d   ? "copy of the rows' x-ranges into every rank's T"
                         : sp->xsplit ? "FFT along X, local"
                                      : "FFT along Y, stores into every rank's T";
        const char* wb = sp->rows2d   ? "FFT along Y, stores into every rank's row buffer"
                         : sp->xsplit ? "FFT along Y, stores into every rank's R"
                                      : "FFT along Z, stores into every rank's staging buffer";
        const char* wc = sp->rows2d ? "FFT along X, local" : sp->xsplit ? "FFT along Z, local" : "FFT along X, local";
        std::vector<std::string> a = items("A", wa, sp->passA), b = items("B", wb, sp->passB), c = items("C", wc, sp->passC);
        o << "  bar0 [shape=box,label=\"barrier (one-word all-reduce over " << sp->P << " ranks)\"];\n"
          << "  bar1 [shape=box,label=\"barrier (one-word all-reduce over " << sp->P << " ranks)\"];\n";
        auto chain = [&](const std::vector<std::string>& ids, const std::string& from, const std::string& to) {
            std::string prev = from;
            for(const auto& id : ids)
            {
                if(!prev.empty())
                    o << "  " << prev << " -> " << id << ";\n";
                prev = id;
            }
            if(!to.empty() && !prev.empty())
                o << "  " << prev << " -> " << to << ";\n";
        };
        chain(a, "", "bar0");
        chain(b, "bar0", "bar1");
        chain(c, "bar1", "");
        o << "}";
        return o.str();
    }

    void multi_device_error_flags(const rocfft_plan_t* plan, std::vector<const int*>& out)
    {
        if(multi_device_kind(plan) == 1)
            return gather_scatter_error_flags(plan, out);
        auto* sp = static_cast<const SlabPlan*>(plan->mgpu);
        if(!sp)
            return;
        for(auto* v : {&sp->passA, &sp->passB, &sp->passC})
            for(auto& c : *v)
                if(c && c->dev_error)
                    out.push_back(c->dev_error);
        // sums of the ranks' failure flags, carried by the two phase barriers
        if(sp->p2p && sp->bar && sp->P > 1)
            for(int i = 0; i < 2; ++i)
                out.push_back(sp->bar + 8 + i);
    }

    rocfft_status execute_multi_device_plan(rocfft_plan_t*                 plan,
                                            void* const*                   in,
                                            void* const*                   out,
                                            const rocfft_execution_info_t* info)
    {
        if(multi_device_kind(plan) == 1)
            return execute_gather_scatter_plan(plan, in, out, info);
        auto* sp = static_cast<SlabPlan*>(plan->mgpu);
        if(!sp || (!sp->comm_stream && !sp->p2p))
            return rocfft_status_failure;
        NcclApi& N = nccl();
        if(sp->p2p)
        {
            // Fused compute + exchange: pass A stores every destination's block straight into
            // that rank's receive buffer over NVLink; a stream-ordered all-reduce of one word is
            // the barrier that tells every rank its buffer is complete; same for pass B; pass C
            // is local.  The barrier at the end of a phase also guarantees that nobody still
            // reads a buffer when the next call (or phase) overwrites it.
            cudaStream_t s = info->stream;
            auto barrier = [&](int slot) {
                return N.AllReduce(sp->bar + slot, sp->bar + 8 + slot, 1, ncclInt, ncclSum, sp->comm, s) == ncclSuccess;
            };
            // ROCFFT_B200_MGPU_TIMING=1: print the device time of every phase (synchronises)
            static const bool timing = getenv("ROCFFT_B200_MGPU_TIMING") != nullptr;
            cudaEvent_t       ev[6]  = {};
            auto mark = [&](int i) {
                if(timing)
                {
                    cudaEventCreate(&ev[i]);
                    cudaEventRecord(ev[i], s);
                }
            };
            // A rank that fails locally (bad argument, launch error) must not leave the others
            // waiting in a barrier that it never enters: the passes are skipped from the failure
            // on, but BOTH barriers are still enqueued, and each carries the sum of the ranks'
            // failure flags, which lands in every rank's barrier words (bar[8], bar[9]).  Those
            // words are part of what b200fft_plan_device_error reports, so every rank can learn
            // that the step's result is not valid; the failing rank itself returns the failure.
            rocfft_status st = rocfft_status_success;
            if(!in || !in[0] || (plan->placement == rocfft_placement_notinplace && (!out || !out[0])))
                st = rocfft_status_failure;
            auto flag = [&](int slot) {
                // barrier word of this rank: 0 while healthy, nonzero after a local failure
                cudaMemsetAsync(sp->bar + slot, st == rocfft_status_success ? 0 : 1, sizeof(int), s);
            };
            mark(0);
            if(st == rocfft_status_success)
                st = execute_core(*sp->passA[0], in, out, nullptr, s);
            mark(1);
            if(sp->P > 1)
            {
                // (single-transpose plan: this barrier also tells every rank that the others have finished
                // reading their R of the previous call, which pass B is about to overwrite)
                flag(0);
                if(!barrier(0))
                    return rocfft_status_failure; // the communicator itself is broken: nothing more can be enqueued
            }
            mark(2);
            if(st == rocfft_status_success)
                st = execute_core(*sp->passB[0], in, out, nullptr, s);
            mark(3);
            if(sp->P > 1)
            {
                flag(1);
                if(!barrier(1))
                    return rocfft_status_failure;
            }
            mark(4);
            if(st == rocfft_status_success)
                st = execute_core(*sp->passC[0], in, out, nullptr, s);
            mark(5);
            if(timing)
            {
                cudaStreamSynchronize(s);
                float ms[5];
                for(int i = 0; i < 5; ++i)
                    cudaEventElapsedTime(&ms[i], ev[i], ev[i + 1]);
                fprintf(stderr,
                        "[rank %d] pass A %.3f ms | barrier %.3f | pass B %.3f | barrier %.3f | pass C %.3f\n",
                        sp->rank, ms[0], ms[1], ms[2], ms[3], ms[4]);
                for(auto& e : ev)
                    cudaEventDestroy(e);
            }
            return st;
        }
        if(!info->workBuffer || info->workBufferSize < sp->work_bytes)
            return rocfft_status_invalid_work_buffer; // the NCCL exchange needs a caller-owned work buffer
        char*        work = static_cast<char*>(info->workBuffer);
        cudaStream_t cs   = info->stream; // compute
        cudaStream_t ns   = sp->comm_stream; // NCCL
        const int    k = sp->chunks, P = sp->P;
        // the exchange stream must not run ahead of work already queued on the caller's stream
        cudaEventRecord(sp->ev_start, cs);
        cudaStreamWaitEvent(ns, sp->ev_start, 0);

        std::vector<size_t> soff(P), roff(P);
        auto exchange = [&](const char* send_base, char* recv_base, bool first, int c) -> bool {
            size_t blk = 0;
            slab_exchange_offsets(P, k, sp->slab_bytes, first ? 1 : 0, c, soff.data(), roff.data(), &blk);
            if(N.GroupStart() != ncclSuccess)
                return false;
            for(int q = 0; q < P; ++q)
            {
                if(N.Send(send_base + soff[q], blk, ncclChar, q, sp->comm, ns) != ncclSuccess)
                    return false;
                if(N.Recv(recv_base + roff[q], blk, ncclChar, q, sp->comm, ns) != ncclSuccess)
                    return false;
            }
            return N.GroupEnd() == ncclSuccess;
        };

        // pass A per chunk, exchange #1 per chunk
        for(int c = 0; c < k; ++c)
        {
            rocfft_status st = execute_core(*sp->passA[c], in, out, work, cs);
            if(st != rocfft_status_success)
                return st;
            cudaEventRecord(sp->evA[c], cs);
            cudaStreamWaitEvent(ns, sp->evA[c], 0);
            if(!exchange(work + sp->off_s, work + sp->off_r, true, c))
                return rocfft_status_failure;
        }
        cudaEventRecord(sp->ev_all, ns);
        cudaStreamWaitEvent(cs, sp->ev_all, 0);
        // pass B per chunk, exchange #2 per chunk
        for(int c = 0; c < k; ++c)
        {
            rocfft_status st = execute_core(*sp->passB[c], in, out, work, cs);
            if(st != rocfft_status_success)
                return st;
            cudaEventRecord(sp->evB[c], cs);
            cudaStreamWaitEvent(ns, sp->evB[c], 0);
            if(!exchange(work + sp->off_s, work + sp->off_r2, false, c))
                return rocfft_status_failure;
            cudaEventRecord(sp->evX[c], ns);
        }
        // pass C per chunk as its data arrives
        for(int c = 0; c < k; ++c)
        {
            cudaStreamWaitEvent(cs, sp->evX[c], 0);
            rocfft_status st = execute_core(*sp->passC[c], in, out, work, cs);
            if(st != rocfft_status_success)
                return st;
        }
        return rocfft_status_success;
    }

    // ---- communicator helpers exported through rocfft_b200_ext.h ----
    int nccl_unique_id(void* out128)
    {
        NcclApi& N = nccl();
        if(!N.ok)
            return 1;
        ncclUniqueId id;
        if(N.GetUniqueId(&id) != ncclSuccess)
            return 2;
        memcpy(out128, &id, sizeof id);
        return 0;
    }
    int nccl_comm_create(int nranks, int rank, const void* id128, void** comm_out)
    {
        NcclApi& N = nccl();
        if(!N.ok)
            return 1;
        ncclUniqueId id;
        memcpy(&id, id128, sizeof id);
        ncclComm_t c = nullptr;
        if(N.CommInitRank(&c, nranks, id, rank) != ncclSuccess)
            return 2;
        *comm_out = c;
        return 0;
    }
    int nccl_comm_destroy(void* comm)
    {
        NcclApi& N = nccl();
        if(!N.ok)
            return 1;
        return N.CommDestroy((ncclComm_t)comm) == ncclSuccess ? 0 : 2;
    }
}
