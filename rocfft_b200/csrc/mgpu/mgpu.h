// Multi-device layer: bricks, fields, slab decomposition and the global
// transpose over NCCL / NVLink.
//
// Role in the reference: library/src/plan.cpp:490-696 (fields and bricks),
// :1244-2358 (gather/scatter plans, the optimised multi-device plan and the
// global transpose) and library/src/tree_node.cpp:473-928 (communication ops).
#pragma once
#include "../plan/plan.h"
#include <nccl.h>
#include <vector>

namespace b200fft
{
    // NCCL is resolved at run time so that the library loads (and everything
    // single-GPU works) on machines without it.
    struct NcclApi
    {
        void* handle = nullptr;
        ncclResult_t (*GetUniqueId)(ncclUniqueId*)                                          = nullptr;
        ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int)                    = nullptr;
        ncclResult_t (*CommDestroy)(ncclComm_t)                                              = nullptr;
        ncclResult_t (*CommCount)(const ncclComm_t, int*)                                    = nullptr;
        ncclResult_t (*CommUserRank)(const ncclComm_t, int*)                                 = nullptr;
        ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
        ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t)   = nullptr;
        ncclResult_t (*GroupStart)()                                                         = nullptr;
        ncclResult_t (*GroupEnd)()                                                           = nullptr;
        ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t)
            = nullptr;
        ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t)
            = nullptr;
        const char* (*GetErrorString)(ncclResult_t) = nullptr;
        bool ok                                     = false;
    };

    NcclApi& nccl();

    // plan->mgpu points at one of two plan kinds; both start with this header
    struct MultiDeviceHeader
    {
        int kind; // 0: slab plan over an NCCL communicator (mgpu.cpp), 1: gather / scatter plan (gather_scatter.cpp)
    };
    inline int multi_device_kind(const rocfft_plan_t* plan)
    {
        return plan->mgpu ? static_cast<const MultiDeviceHeader*>(plan->mgpu)->kind : -1;
    }

    // gather / scatter plans: any brick layout of a single process (gather_scatter.cpp)
    void          build_gather_scatter_plan(rocfft_plan_t* plan);
    void          destroy_gather_scatter_plan(rocfft_plan_t* plan);
    size_t        gather_scatter_work_bytes(const rocfft_plan_t* plan);
    std::string   describe_gather_scatter_plan(const rocfft_plan_t* plan);
    void          gather_scatter_error_flags(const rocfft_plan_t* plan, std::vector<const int*>& out);
    rocfft_status execute_gather_scatter_plan(rocfft_plan_t*                 plan,
                                              void* const*                   in,
                                              void* const*                   out,
                                              const rocfft_execution_info_t* info);

    // builds plan->mgpu from the in/out fields of the description; throws on
    // malformed fields (std::runtime_error) so that creation reports failure
    void          build_multi_device_plan(rocfft_plan_t* plan);
    void          destroy_multi_device_plan(rocfft_plan_t* plan);
    size_t        multi_device_work_bytes(const rocfft_plan_t* plan);
    std::string   describe_multi_device_plan(const rocfft_plan_t* plan);
    // device error flags (PlanCore::dev_error) of every local pass of the plan; null entries skipped
    void          multi_device_error_flags(const rocfft_plan_t* plan, std::vector<const int*>& out);
    // the plan's items (local FFT passes, barriers, copies) and their order as a graphviz digraph: graph log layer
    std::string   multi_device_plan_graph(const rocfft_plan_t* plan);
    rocfft_status execute_multi_device_plan(rocfft_plan_t*                 plan,
                                            void* const*                   in,
                                            void* const*                   out,
                                            const rocfft_execution_info_t* info);

    // schedule of one chunk of one exchange (pure host arithmetic; see mgpu.cpp)
    void slab_exchange_offsets(int     ranks,
                               int     chunks,
                               size_t  slab_bytes,
                               int     first,
                               int     c,
                               size_t* send_off,
                               size_t* recv_off,
                               size_t* block_bytes);

    // where rank `rank` of `ranks` stores into every peer's buffers in a row-slab rank-2 plan (byte offsets):
    // first phase: its rows of the peer's T[y][x_local]; second phase: its columns of the peer's [y_local][x]
    void rows2d_exchange_offsets(int ranks, int rank, size_t nx, size_t ny, size_t elem_bytes, size_t* first_off, size_t* second_off);

    // NCCL communicator helpers (0 on success)
    int nccl_unique_id(void* out128);
    int nccl_comm_create(int nranks, int rank, const void* id128, void** comm_out);
    int nccl_comm_destroy(void* comm);
}
