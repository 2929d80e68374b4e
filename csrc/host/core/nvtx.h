// NVTX ranges for the host runtime: a scope object, a range macro and a thread-naming macro, as the reference has around
// its signal operations (NvtxScope / NVTX_RANGE / NVTX_THREAD, dlslime/csrc/device/cuda/nvtx_helper.h:17-38 in the
// reference). NVTX 3 is header-only and costs one pointer test per call when no tool is attached. Where the CUDA toolkit's
// headers are not on the include path the macros expand to nothing, so the runtime builds without CUDA.
#pragma once

#include <cstdint>
#include <unistd.h>
#include <sys/syscall.h>

#if defined(__has_include)
#if __has_include(<nvtx3/nvToolsExt.h>) && !defined(SLIME_NO_NVTX)
#define SLIME_HAVE_NVTX 1
#include <nvtx3/nvToolsExt.h>
#endif
#endif

namespace slime {

// ARGB colours of the ranges, by kind of work.
constexpr uint32_t kNvtxSignal = 0xFF2E86C1u;  // stream <-> engine signalling
constexpr uint32_t kNvtxPost   = 0xFF28B463u;  // posting work to a transport
constexpr uint32_t kNvtxWait   = 0xFFCA6F1Eu;  // waiting for completions

#ifdef SLIME_HAVE_NVTX
class NvtxScope {
public:
    NvtxScope(const char* name, uint32_t argb)
    {
        nvtxEventAttributes_t a{};
        a.version       = NVTX_VERSION;
        a.size          = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
        a.colorType     = NVTX_COLOR_ARGB;
        a.color         = argb;
        a.messageType   = NVTX_MESSAGE_TYPE_ASCII;
        a.message.ascii = name;
        nvtxRangePushEx(&a);
    }
    ~NvtxScope() { nvtxRangePop(); }
    NvtxScope(const NvtxScope&)            = delete;
    NvtxScope& operator=(const NvtxScope&) = delete;
};
inline void nvtx_name_this_thread(const char* name)
{
    nvtxNameOsThreadA(static_cast<uint32_t>(::syscall(SYS_gettid)), name);
}
inline constexpr bool kNvtxCompiledIn = true;
#define SLIME_NVTX_CAT2(a, b) a##b
#define SLIME_NVTX_CAT(a, b) SLIME_NVTX_CAT2(a, b)
#define SLIME_NVTX_RANGE(name, argb) ::slime::NvtxScope SLIME_NVTX_CAT(slime_nvtx_scope_, __LINE__)(name, argb)
#define SLIME_NVTX_THREAD(name) ::slime::nvtx_name_this_thread(name)
#else
inline constexpr bool kNvtxCompiledIn = false;
#define SLIME_NVTX_RANGE(name, argb) ((void)0)
#define SLIME_NVTX_THREAD(name) ((void)0)
#endif

}  // namespace slime
