// The verbs operations the RDMA transport needs, as an interface with two providers:
//
//   * "ibverbs"   libibverbs loaded with dlopen at run time (no link-time or header dependency),
//   * "loopback"  a software reliable-connected fabric inside the process: queue pairs, memory keys,
//                 receive queues, completion queues, RNR back-off, access checks and error/flush
//                 semantics, executed by an engine thread. Every layer above (context, channel,
//                 endpoint, worker) runs unchanged on it, which is how they are tested on hosts
//                 without a NIC.
//
// SLIME_RDMA_PROVIDER=ibverbs|loopback picks one; the default is ibverbs when the library loads and
// has at least one device, else loopback is available only on request.
//
// The structs are the transport's own; the ibverbs provider converts to the library's layout.
// Role in the reference: ibv_* calls made directly in dlslime/csrc/engine/rdma/rdma_context.cpp,
// rdma_channel.cpp and memory_pool.cpp (in the reference).
#pragma once

#include <array>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace slime {
namespace rdma {

enum class LinkLayer : int { UNKNOWN = 0, IB = 1, ETHERNET = 2 };

struct DeviceAttr {
    int max_cqe        = 0;
    int max_qp_wr      = 0;
    int max_sge        = 0;
    int max_qp_rd_atom = 0;
    int phys_port_cnt  = 1;
};

struct PortAttr {
    bool      active      = false;
    uint16_t  lid         = 0;
    int       active_mtu  = 3;  // verbs enum: 1=256 ... 5=4096
    int       gid_tbl_len = 0;
    LinkLayer link_layer  = LinkLayer::UNKNOWN;
};

using Gid = std::array<uint8_t, 16>;

struct Sge {
    uint64_t addr   = 0;
    uint32_t length = 0;
    uint32_t lkey   = 0;
};

enum class WrOp : int { WRITE = 0, WRITE_WITH_IMM = 1, SEND = 2, SEND_WITH_IMM = 3, READ = 4 };

struct SendWr {
    uint64_t wr_id       = 0;
    Sge      sge;
    WrOp     op          = WrOp::WRITE;
    bool     signaled    = false;
    bool     inline_data = false;
    uint32_t imm         = 0;
    uint64_t remote_addr = 0;
    uint32_t rkey        = 0;
};

struct RecvWr {
    uint64_t wr_id = 0;
    Sge      sge;
};

// Completion status values follow the verbs numbering for the ones that matter to callers.
enum WcStatus : int { WC_SUCCESS = 0, WC_LOC_PROT_ERR = 4, WC_WR_FLUSH_ERR = 5, WC_REM_ACCESS_ERR = 10, WC_RETRY_EXC_ERR = 12, WC_RNR_RETRY_EXC_ERR = 13, WC_GENERAL_ERR = 21 };
enum class WcOp : int { SEND = 0, WRITE = 1, READ = 2, RECV = 128, RECV_WITH_IMM = 129 };

struct Completion {
    uint64_t wr_id    = 0;
    int      status   = WC_SUCCESS;
    WcOp     op       = WcOp::SEND;
    uint32_t imm      = 0;
    bool     has_imm  = false;
    uint32_t byte_len = 0;
    uint32_t qp_num   = 0;
};

struct MrKeys {
    uint64_t handle = 0;  // provider object
    uint32_t lkey   = 0;
    uint32_t rkey   = 0;
};

struct QpCaps {
    int max_send_wr = 4096;
    int max_recv_wr = 4096;
    int max_inline  = 0;
};

struct QpRoute {  // what RTR / RTS need about the two ends
    uint32_t dest_qpn           = 0;
    uint32_t dest_psn           = 0;  // rq_psn: first PSN the peer will send
    uint32_t local_psn          = 0;  // sq_psn
    int      mtu                = 3;
    Gid      dest_gid{};
    int      sgid_index         = 0;
    uint16_t dest_lid           = 0;
    bool     is_global          = false;  // RoCE (GRH) vs InfiniBand (LID) addressing
    int      port               = 1;
    int      service_level      = 0;
    int      max_rd_atomic      = 16;
    int      max_dest_rd_atomic = 16;
    int      min_rnr_timer      = 0x20;
    int      timeout            = 14;
    int      retry_cnt          = 7;
    int      rnr_retry          = 7;
};

// One opened device. Handles are opaque provider objects; all calls are thread-safe the way the
// verbs specification makes them (post / poll on different queue pairs or from different threads).
class VerbsDevice {
public:
    virtual ~VerbsDevice() = default;

    virtual std::string name() const                                 = 0;
    virtual DeviceAttr  query_device()                               = 0;
    virtual PortAttr    query_port(int port)                         = 0;
    virtual bool        query_gid(int port, int index, Gid& out)     = 0;
    // Index of a RoCE v2 / IPv4-mapped GID on the port, or -1.
    virtual int         find_roce_v2_gid(int port, int gid_tbl_len)  = 0;

    virtual uint64_t alloc_pd()                                                     = 0;
    virtual void     dealloc_pd(uint64_t pd)                                        = 0;
    virtual bool     reg_mr(uint64_t pd, uintptr_t addr, uint64_t len, MrKeys& out) = 0;
    virtual void     dereg_mr(uint64_t mr_handle)                                   = 0;

    virtual uint64_t create_cq(int depth)                                      = 0;
    virtual void     destroy_cq(uint64_t cq)                                   = 0;
    virtual int      poll_cq(uint64_t cq, int max_entries, Completion* out)    = 0;
    // Arms the completion queue and sleeps until an event or the timeout; true if an event came.
    virtual bool     wait_cq_event(uint64_t cq, int timeout_ms)                = 0;

    virtual uint64_t create_qp(uint64_t pd, uint64_t cq, const QpCaps& caps, uint32_t& qp_num_out) = 0;
    virtual void     destroy_qp(uint64_t qp)                                                       = 0;
    virtual int      qp_to_init(uint64_t qp, int port)                                             = 0;
    virtual int      qp_to_rtr(uint64_t qp, const QpRoute& route)                                  = 0;
    virtual int      qp_to_rts(uint64_t qp, const QpRoute& route)                                  = 0;
    // Posts wrs[0..n) in order as one chain. Returns 0, or an errno-style code with *n_posted set.
    virtual int      post_send(uint64_t qp, const SendWr* wrs, int n, int* n_posted)               = 0;
    virtual int      post_recv(uint64_t qp, const RecvWr* wrs, int n, int* n_posted)               = 0;
};

class VerbsProvider {
public:
    virtual ~VerbsProvider() = default;
    virtual std::string                  provider_name() const          = 0;
    virtual std::vector<std::string>     list_devices()                 = 0;
    virtual std::shared_ptr<VerbsDevice> open_device(const std::string& name) = 0;
};

// nullptr when the provider cannot be used (library missing, no devices) with the reason in *why.
VerbsProvider* ibverbs_provider(std::string* why = nullptr);
VerbsProvider* loopback_provider();
// The provider selected by SLIME_RDMA_PROVIDER (see the top of this file); nullptr if none.
VerbsProvider* default_provider(std::string* why = nullptr);

// Test hooks of the loopback fabric: the next `count` work requests of the given kind complete with
// `status` (and move the queue pair to the error state, flushing what follows, as hardware does).
void loopback_inject_error(WrOp op, int status, int count);
// Total work requests executed / receive-not-ready back-offs seen since the start.
uint64_t loopback_executed_wrs();
uint64_t loopback_rnr_events();

}  // namespace rdma
}  // namespace slime
