// Ascend Direct endpoint: interface only. The reference drives Huawei's ADXL engine
// (dlslime/csrc/engine/ascend_direct/ascend_direct_endpoint.h:24-89 in the reference);
// that SDK does not exist on NVIDIA hosts, so this class keeps the method surface and the
// endpoint_info / mr_info JSON shape ({host, port, mr_info:{name:{name,addr,offset,length}}})
// and reports "not available" from every data-path call.
#pragma once

#include <map>
#include <optional>
#include <stdexcept>
#include <string>

#include "core/json.hpp"

namespace slime {

class AscendDirectEndpoint {
public:
    int init(const std::string& host, int port)
    {
        host_ = host;
        port_ = port;
        return 0;
    }
    int32_t register_memory_region(uintptr_t addr, size_t offset, size_t length, const std::optional<std::string>& name)
    {
        Json e      = Json::object();
        const std::string n = name ? *name : "auto_" + std::to_string(addr + offset);
        e["name"]   = n;
        e["addr"]   = static_cast<unsigned long long>(addr);
        e["offset"] = static_cast<unsigned long long>(offset);
        e["length"] = static_cast<unsigned long long>(length);
        auto it     = handles_.find(n);
        if (it == handles_.end()) it = handles_.emplace(n, static_cast<int32_t>(handles_.size())).first;
        mr_[n] = e;
        return it->second;
    }
    int32_t get_mr_handle(const std::string& name) const
    {
        auto it = handles_.find(name);
        return it == handles_.end() ? -1 : it->second;
    }
    Json mr_info() const { return mr_; }
    Json endpoint_info() const
    {
        Json j       = Json::object();
        j["host"]    = host_;
        j["port"]    = port_;
        j["mr_info"] = mr_;
        return j;
    }
    [[noreturn]] static void unavailable(const char* what)
    {
        throw std::runtime_error(std::string("AscendDirectEndpoint.") + what + ": the Ascend ADXL transport is not available in this build (NVIDIA B200 target)");
    }
    int  connect(const Json&) { unavailable("connect"); }
    int  disconnect(const Json&) { unavailable("disconnect"); }
    void read() { unavailable("read"); }

private:
    std::string                    host_;
    int                            port_ = 0;
    Json                           mr_   = Json::object();
    std::map<std::string, int32_t> handles_;
};

}  // namespace slime
