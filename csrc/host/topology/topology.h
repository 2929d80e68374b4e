// Host topology discovery: RDMA NICs from sysfs, NVIDIA GPUs from procfs, and a TCP
// pseudo-link so that CPU-only hosts can still register with the control plane.
// Output schema (version 1) is the one PeerAgent publishes, as in the reference
// (dlslime/csrc/topology.cpp:229-296 in the reference):
//   {schema_version, host:{hostname,address}, nics:[{name,health,numa_node,pci_bus_id,
//    ports:[{port,state,link_type,active_mtu?}]}], accelerators:[], memory_keys:[], topology_epoch}
// sysfs_root / procfs_root / devices can be injected, which is how the tests build fake trees.
#pragma once

#include <optional>
#include <string>
#include <vector>

#include "core/json.hpp"

namespace slime {
namespace topology {

struct Options {
    std::optional<std::string>              preferred_device;
    int                                     ib_port = 1;
    std::optional<std::string>              preferred_link_type;
    std::string                             sysfs_root  = "/sys";
    std::string                             procfs_root = "/proc";
    std::optional<std::vector<std::string>> devices;
    bool allow_software_links = false;  // add a "tcp0" pseudo NIC when no RDMA device exists instead of throwing
};

std::string normalize_link_type(const std::string& raw);   // Ethernet/roce -> RoCE, InfiniBand/ib -> IB, tcp -> TCP, nvlink -> NVLink
std::string normalize_port_state(const std::string& raw);  // "4: ACTIVE\n" -> ACTIVE
std::vector<std::string> list_rdma_devices(const std::string& sysfs_root);
Json                     list_accelerators(const std::string& procfs_root);
Json                     discover(const Options& opt);
int                      numa_node_of(const std::string& device, const std::string& sysfs_root = "/sys");

}  // namespace topology
}  // namespace slime
