#include "topology/topology.h"

#include <algorithm>
#include <cctype>
#include <chrono>
#include <filesystem>
#include <fstream>
#include <sstream>
#include <stdexcept>

#include <arpa/inet.h>
#include <ifaddrs.h>
#include <netinet/in.h>
#include <unistd.h>

#include "core/env.h"

namespace fs = std::filesystem;

namespace slime {
namespace topology {

namespace {

std::string strip(const std::string& s)
{
    size_t b = 0, e = s.size();
    while (b < e && std::isspace(static_cast<unsigned char>(s[b]))) ++b;
    while (e > b && std::isspace(static_cast<unsigned char>(s[e - 1]))) --e;
    return s.substr(b, e - b);
}

std::string lower(std::string s)
{
    for (auto& c : s) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
    return s;
}

bool read_file(const fs::path& p, std::string& out)
{
    std::ifstream f(p);
    if (!f) return false;
    std::stringstream ss;
    ss << f.rdbuf();
    out = strip(ss.str());
    return true;
}

fs::path ib_dir(const std::string& sysfs_root)
{
    return fs::path(sysfs_root) / "class" / "infiniband";
}

Json local_host()
{
    char name[256] = {0};
    gethostname(name, sizeof(name) - 1);
    std::string address = "127.0.0.1";
    ifaddrs*    ifs     = nullptr;
    if (getifaddrs(&ifs) == 0) {
        for (ifaddrs* it = ifs; it != nullptr; it = it->ifa_next) {
            if (!it->ifa_addr || it->ifa_addr->sa_family != AF_INET) continue;
            char buf[INET_ADDRSTRLEN];
            inet_ntop(AF_INET, &reinterpret_cast<sockaddr_in*>(it->ifa_addr)->sin_addr, buf, sizeof(buf));
            if (std::string(buf).rfind("127.", 0) == 0) continue;
            address = buf;
            break;
        }
        freeifaddrs(ifs);
    }
    Json h       = Json::object();
    h["hostname"] = std::string(name[0] ? name : "localhost");
    h["address"]  = address;
    return h;
}

Json read_port(const std::string& dev, int port, const std::string& sysfs_root)
{
    Json p         = Json::object();
    p["port"]      = port;
    p["state"]     = "UNKNOWN";
    p["link_type"] = "UNKNOWN";
    const fs::path root = ib_dir(sysfs_root) / dev / "ports" / std::to_string(port);
    std::string    v;
    if (read_file(root / "state", v)) p["state"] = normalize_port_state(v);
    if (read_file(root / "link_layer", v)) p["link_type"] = normalize_link_type(v);
    if (read_file(root / "active_mtu", v)) {
        // "4096" or "5: 4096" depending on the driver
        const size_t colon = v.find(':');
        const std::string num = strip(colon == std::string::npos ? v : v.substr(colon + 1));
        char* end = nullptr;
        long  mtu = std::strtol(num.c_str(), &end, 10);
        if (end != num.c_str()) p["active_mtu"] = static_cast<long long>(mtu);
    }
    return p;
}

}  // namespace

std::string normalize_link_type(const std::string& raw)
{
    const std::string v = strip(raw), l = lower(v);
    if (l == "ethernet" || l == "roce") return "RoCE";
    if (l == "infiniband" || l == "ib") return "IB";
    if (l == "tcp") return "TCP";
    if (l == "nvlink") return "NVLink";
    return v.empty() ? "UNKNOWN" : v;
}

std::string normalize_port_state(const std::string& raw)
{
    std::string v = strip(raw);
    const size_t colon = v.find(':');
    if (colon != std::string::npos) v = strip(v.substr(colon + 1));
    for (auto& c : v) c = static_cast<char>(std::toupper(static_cast<unsigned char>(c)));
    return v.empty() ? "UNKNOWN" : v;
}

std::vector<std::string> list_rdma_devices(const std::string& sysfs_root)
{
    std::vector<std::string> out;
    std::error_code          ec;
    const fs::path           root = ib_dir(sysfs_root);
    if (fs::exists(root, ec)) {
        for (const auto& e : fs::directory_iterator(root, ec)) out.push_back(e.path().filename().string());
    }
    const auto visible = get_env<std::vector<std::string>>("SLIME_VISIBLE_DEVICES", {});
    if (!visible.empty())
        out.erase(std::remove_if(out.begin(), out.end(),
                                 [&](const std::string& d) { return std::find(visible.begin(), visible.end(), d) == visible.end(); }),
                  out.end());
    std::sort(out.begin(), out.end());
    return out;
}

int numa_node_of(const std::string& device, const std::string& sysfs_root)
{
    std::error_code ec;
    const fs::path  dev = fs::weakly_canonical(ib_dir(sysfs_root) / device / "device", ec);
    std::string     v;
    if (!ec && read_file(dev / "numa_node", v)) {
        char* end = nullptr;
        long  n   = std::strtol(v.c_str(), &end, 10);
        if (end != v.c_str()) return static_cast<int>(n);
    }
    return -1;
}

Json list_accelerators(const std::string& procfs_root)
{
    // /proc/driver/nvidia/gpus/<pci bus id>/information holds "Model:" and "GPU UUID:" lines
    Json            out = Json::array();
    std::error_code ec;
    const fs::path  root = fs::path(procfs_root) / "driver" / "nvidia" / "gpus";
    if (!fs::exists(root, ec)) return out;
    std::vector<std::string> ids;
    for (const auto& e : fs::directory_iterator(root, ec)) ids.push_back(e.path().filename().string());
    std::sort(ids.begin(), ids.end());
    int ordinal = 0;
    for (const auto& id : ids) {
        Json a          = Json::object();
        a["ordinal"]    = ordinal++;
        a["pci_bus_id"] = id;
        a["kind"]       = "cuda";
        a["link_type"]  = "NVLink";
        std::ifstream f(root / id / "information");
        std::string   line;
        while (std::getline(f, line)) {
            const size_t colon = line.find(':');
            if (colon == std::string::npos) continue;
            const std::string key = strip(line.substr(0, colon)), val = strip(line.substr(colon + 1));
            if (key == "Model") a["model"] = val;
            else if (key == "GPU UUID") a["uuid"] = val;
        }
        out.push_back(a);
    }
    return out;
}

Json discover(const Options& opt)
{
    std::vector<std::string> devices = opt.devices ? *opt.devices : list_rdma_devices(opt.sysfs_root);
    if (opt.preferred_device && !opt.preferred_device->empty()) {
        // the preferred device moves to the front, but only if it is in the visible set
        auto it = std::find(devices.begin(), devices.end(), *opt.preferred_device);
        if (it != devices.end()) std::rotate(devices.begin(), it, it + 1);
    }
    Json nics = Json::array();
    if (devices.empty()) {
        if (!opt.allow_software_links) throw std::runtime_error("No RDMA devices available");
        Json port         = Json::object();
        port["port"]      = opt.ib_port;
        port["state"]     = "ACTIVE";
        port["link_type"] = "TCP";
        Json nic          = Json::object();
        nic["name"]       = "tcp0";
        nic["health"]     = "AVAILABLE";
        nic["numa_node"]  = -1;
        nic["pci_bus_id"] = "";
        Json ports        = Json::array();
        ports.push_back(port);
        nic["ports"] = ports;
        nics.push_back(nic);
    }
    for (const auto& dev : devices) {
        Json port = read_port(dev, opt.ib_port, opt.sysfs_root);
        if (port["link_type"].as_string() == "UNKNOWN")
            port["link_type"] = opt.preferred_link_type ? normalize_link_type(*opt.preferred_link_type) : std::string("UNKNOWN");
        if (port["state"].as_string() == "UNKNOWN") port["state"] = "ACTIVE";
        std::string     bdf;
        std::error_code ec;
        const fs::path  link = ib_dir(opt.sysfs_root) / dev / "device";
        if (fs::exists(link, ec)) bdf = fs::weakly_canonical(link, ec).filename().string();
        Json nic          = Json::object();
        nic["name"]       = dev;
        nic["health"]     = port["state"].as_string() == "ACTIVE" ? "AVAILABLE" : "DEGRADED";
        nic["numa_node"]  = numa_node_of(dev, opt.sysfs_root);
        nic["pci_bus_id"] = bdf;
        Json ports        = Json::array();
        ports.push_back(port);
        nic["ports"] = ports;
        nics.push_back(nic);
    }
    Json out              = Json::object();
    out["schema_version"] = 1;
    out["host"]           = local_host();
    out["nics"]           = nics;
    out["accelerators"]   = list_accelerators(opt.procfs_root);
    out["memory_keys"]    = Json::array();
    out["topology_epoch"] = static_cast<long long>(
        std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count());
    return out;
}

}  // namespace topology
}  // namespace slime
