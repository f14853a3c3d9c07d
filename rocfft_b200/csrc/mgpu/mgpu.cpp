#include "mgpu.h"
#include <stdexcept>

namespace b200fft
{
    void build_multi_device_plan(rocfft_plan_t*)
    {
        throw std::runtime_error("multi-device plans are not available yet");
    }
    void destroy_multi_device_plan(rocfft_plan_t*) {}
    std::string describe_multi_device_plan(const rocfft_plan_t*)
    {
        return "";
    }
    size_t multi_device_work_bytes(const rocfft_plan_t*)
    {
        return 0;
    }
    rocfft_status execute_multi_device_plan(rocfft_plan_t*, void* const*, void* const*, const rocfft_execution_info_t*)
    {
        return rocfft_status_failure;
    }
}
