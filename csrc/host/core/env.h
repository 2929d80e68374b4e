// Typed environment lookups with defaults, including comma-separated lists, and the
// runtime knobs of the transfer engines. Same variable names and defaults as the
// reference (dlslime/csrc/env.h:19-57, dlslime/csrc/engine/rdma/rdma_env.h:10-28 in the
// reference) so existing deployments keep their tuning.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <sstream>
#include <string>
#include <type_traits>
#include <vector>

namespace slime {

template<typename T>
T get_env(const char* name, T dflt)
{
    const char* raw = std::getenv(name);
    if (raw == nullptr || *raw == 0) return dflt;
    if constexpr (std::is_same_v<T, std::string>) {
        return std::string(raw);
    }
    else if constexpr (std::is_same_v<T, std::vector<std::string>>) {
        std::vector<std::string> out;
        std::stringstream        ss(raw);
        std::string              item;
        while (std::getline(ss, item, ','))
            if (!item.empty()) out.push_back(item);
        return out;
    }
    else if constexpr (std::is_same_v<T, bool>) {
        std::string s(raw);
        return !(s == "0" || s == "false" || s == "FALSE" || s == "off" || s == "OFF");
    }
    else if constexpr (std::is_floating_point_v<T>) {
        char*  end = nullptr;
        double v   = std::strtod(raw, &end);
        return (end && *end == 0) ? static_cast<T>(v) : dflt;
    }
    else if constexpr (std::is_integral_v<T> || std::is_enum_v<T>) {
        char*     end = nullptr;
        long long v   = std::strtoll(raw, &end, 0);
        return (end && *end == 0) ? static_cast<T>(v) : dflt;
    }
    else {
        static_assert(!sizeof(T), "unsupported type for get_env");
    }
}

struct EngineEnv {
    int                      log_level          = get_env<int>("SLIME_LOG_LEVEL", 0);
    int                      log_mutex          = get_env<int>("SLIME_LOG_MUTEX", 0);
    std::vector<std::string> visible_devices    = get_env<std::vector<std::string>>("SLIME_VISIBLE_DEVICES", {});
    uint64_t                 max_length_per_assignment = get_env<uint64_t>("SLIME_MAX_LENGTH_PER_ASSIGNMENT", 1ull << 30);
    int                      max_send_wr        = get_env<int>("SLIME_MAX_SEND_WR", 4096);
    int                      max_recv_wr        = get_env<int>("SLIME_MAX_RECV_WR", 4096);
    int                      poll_count         = get_env<int>("SLIME_POLL_COUNT", 256);
    int                      max_rd_atomic      = get_env<int>("SLIME_MAX_RD_ATOMIC", 16);
    int                      max_dest_rd_atomic = get_env<int>("SLIME_MAX_DEST_RD_ATOMIC", 16);
    int                      service_level      = get_env<int>("SLIME_SERVICE_LEVEL", 0);
    int                      gid_index          = get_env<int>("SLIME_GID_INDEX", -1);
    int                      qp_num             = get_env<int>("SLIME_QP_NUM", 2);
    int                      cq_num             = get_env<int>("SLIME_CQ_NUM", 1);
    int                      max_cq_depth       = get_env<int>("SLIME_MAX_CQ_DEPTH", 65536);
    int                      agg_qp_num         = get_env<int>("SLIME_AGG_QP_NUM", 1);
    int                      bypass_device_signal = get_env<int>("SLIME_BYPASS_DEVICE_SIGNAL", 1);
    int                      max_msg_fifo_depth = get_env<int>("SLIME_MAX_MSG_FIFO_DEPTH", 1024);
    int                      max_io_fifo_depth  = get_env<int>("SLIME_MAX_IO_FIFO_DEPTH", 2048);
    int                      with_time_trace    = get_env<int>("SLIME_WITH_TIME_TRACE", 1);
};

// Read once, at first use. Tests that shrink queue depths set the variables before importing.
inline const EngineEnv& engine_env()
{
    static const EngineEnv env;
    return env;
}

}  // namespace slime
