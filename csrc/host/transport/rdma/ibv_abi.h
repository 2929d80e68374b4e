// The subset of the libibverbs (rdma-core, ABI version 1) binary interface that the "ibverbs"
// provider uses, declared here because the library is loaded with dlopen and its headers are not a
// build dependency. Layouts are those of the public <infiniband/verbs.h>; only members this
// transport reads or writes are named, the rest is kept as correctly sized fields so offsets match.
// Fast-path calls (post_send, post_recv, poll_cq, req_notify_cq) are function pointers in
// ibv_context::ops, as in the library's own inline wrappers.
#pragma once

#include <cstddef>
#include <cstdint>
#include <pthread.h>

extern "C" {

struct ibv_device;
struct ibv_context;
struct ibv_pd;
struct ibv_mr;
struct ibv_cq;
struct ibv_qp;
struct ibv_srq;
struct ibv_ah;
struct ibv_mw;
struct ibv_comp_channel;
struct ibv_wc;
struct ibv_send_wr;
struct ibv_recv_wr;
struct ibv_mw_bind;

union ibv_gid {
    uint8_t raw[16];
    struct {
        uint64_t subnet_prefix;
        uint64_t interface_id;
    } global;
};

struct ibv_device_attr {
    char     fw_ver[64];
    uint64_t node_guid;
    uint64_t sys_image_guid;
    uint64_t max_mr_size;
    uint64_t page_size_cap;
    uint32_t vendor_id;
    uint32_t vendor_part_id;
    uint32_t hw_ver;
    int      max_qp;
    int      max_qp_wr;
    unsigned device_cap_flags;
    int      max_sge;
    int      max_sge_rd;
    int      max_cq;
    int      max_cqe;
    int      max_mr;
    int      max_pd;
    int      max_qp_rd_atom;
    int      max_ee_rd_atom;
    int      max_res_rd_atom;
    int      max_qp_init_rd_atom;
    int      max_ee_init_rd_atom;
    int      atomic_cap;
    int      max_ee;
    int      max_rdd;
    int      max_mw;
    int      max_raw_ipv6_qp;
    int      max_raw_ethy_qp;
    int      max_mcast_grp;
    int      max_mcast_qp_attach;
    int      max_total_mcast_qp_attach;
    int      max_ah;
    int      max_fmr;
    int      max_map_per_fmr;
    int      max_srq;
    int      max_srq_wr;
    int      max_srq_sge;
    uint16_t max_pkeys;
    uint8_t  local_ca_ack_delay;
    uint8_t  phys_port_cnt;
};

enum { IBV_PORT_ACTIVE = 4 };
enum { IBV_LINK_LAYER_UNSPECIFIED = 0, IBV_LINK_LAYER_INFINIBAND = 1, IBV_LINK_LAYER_ETHERNET = 2 };

struct ibv_port_attr {
    int      state;
    int      max_mtu;
    int      active_mtu;
    int      gid_tbl_len;
    uint32_t port_cap_flags;
    uint32_t max_msg_sz;
    uint32_t bad_pkey_cntr;
    uint32_t qkey_viol_cntr;
    uint16_t pkey_tbl_len;
    uint16_t lid;
    uint16_t sm_lid;
    uint8_t  lmc;
    uint8_t  max_vl_num;
    uint8_t  sm_sl;
    uint8_t  subnet_timeout;
    uint8_t  init_type_reply;
    uint8_t  active_width;
    uint8_t  active_speed;
    uint8_t  phys_state;
    uint8_t  link_layer;
    uint8_t  flags;
    uint16_t port_cap_flags2;
    uint32_t active_speed_ex;
    uint8_t  reserved_tail[32];  // room for members added by newer library versions
};

struct ibv_mr {
    ibv_context* context;
    ibv_pd*      pd;
    void*        addr;
    size_t       length;
    uint32_t     handle;
    uint32_t     lkey;
    uint32_t     rkey;
};

enum { IBV_ACCESS_LOCAL_WRITE = 1, IBV_ACCESS_REMOTE_WRITE = 2, IBV_ACCESS_REMOTE_READ = 4 };

struct ibv_global_route {
    ibv_gid  dgid;
    uint32_t flow_label;
    uint8_t  sgid_index;
    uint8_t  hop_limit;
    uint8_t  traffic_class;
};

struct ibv_ah_attr {
    ibv_global_route grh;
    uint16_t         dlid;
    uint8_t          sl;
    uint8_t          src_path_bits;
    uint8_t          static_rate;
    uint8_t          is_global;
    uint8_t          port_num;
};

struct ibv_qp_cap {
    uint32_t max_send_wr;
    uint32_t max_recv_wr;
    uint32_t max_send_sge;
    uint32_t max_recv_sge;
    uint32_t max_inline_data;
};

enum { IBV_QPT_RC = 2 };

struct ibv_qp_init_attr {
    void*      qp_context;
    ibv_cq*    send_cq;
    ibv_cq*    recv_cq;
    ibv_srq*   srq;
    ibv_qp_cap cap;
    int        qp_type;
    int        sq_sig_all;
};

enum { IBV_QPS_RESET = 0, IBV_QPS_INIT = 1, IBV_QPS_RTR = 2, IBV_QPS_RTS = 3 };

enum {
    IBV_QP_STATE              = 1 << 0,
    IBV_QP_ACCESS_FLAGS       = 1 << 3,
    IBV_QP_PKEY_INDEX         = 1 << 4,
    IBV_QP_PORT               = 1 << 5,
    IBV_QP_AV                 = 1 << 7,
    IBV_QP_PATH_MTU           = 1 << 8,
    IBV_QP_TIMEOUT            = 1 << 9,
    IBV_QP_RETRY_CNT          = 1 << 10,
    IBV_QP_RNR_RETRY          = 1 << 11,
    IBV_QP_RQ_PSN             = 1 << 12,
    IBV_QP_MAX_QP_RD_ATOMIC   = 1 << 13,
    IBV_QP_MIN_RNR_TIMER      = 1 << 15,
    IBV_QP_SQ_PSN             = 1 << 16,
    IBV_QP_MAX_DEST_RD_ATOMIC = 1 << 17,
    IBV_QP_DEST_QPN           = 1 << 20,
};

struct ibv_qp_attr {
    int         qp_state;
    int         cur_qp_state;
    int         path_mtu;
    int         path_mig_state;
    uint32_t    qkey;
    uint32_t    rq_psn;
    uint32_t    sq_psn;
    uint32_t    dest_qp_num;
    unsigned    qp_access_flags;
    ibv_qp_cap  cap;
    ibv_ah_attr ah_attr;
    ibv_ah_attr alt_ah_attr;
    uint16_t    pkey_index;
    uint16_t    alt_pkey_index;
    uint8_t     en_sqd_async_notify;
    uint8_t     sq_draining;
    uint8_t     max_rd_atomic;
    uint8_t     max_dest_rd_atomic;
    uint8_t     min_rnr_timer;
    uint8_t     port_num;
    uint8_t     timeout;
    uint8_t     retry_cnt;
    uint8_t     rnr_retry;
    uint8_t     alt_port_num;
    uint8_t     alt_timeout;
    uint32_t    rate_limit;
};

struct ibv_sge {
    uint64_t addr;
    uint32_t length;
    uint32_t lkey;
};

enum { IBV_WR_RDMA_WRITE = 0, IBV_WR_RDMA_WRITE_WITH_IMM = 1, IBV_WR_SEND = 2, IBV_WR_SEND_WITH_IMM = 3, IBV_WR_RDMA_READ = 4 };
enum { IBV_SEND_SIGNALED = 1 << 1, IBV_SEND_INLINE = 1 << 3 };

struct ibv_send_wr {
    uint64_t     wr_id;
    ibv_send_wr* next;
    ibv_sge*     sg_list;
    int          num_sge;
    int          opcode;
    unsigned     send_flags;
    uint32_t     imm_data;  // big endian on the wire; the provider converts
    union {
        struct {
            uint64_t remote_addr;
            uint32_t rkey;
        } rdma;
        struct {
            uint64_t remote_addr;
            uint64_t compare_add;
            uint64_t swap;
            uint32_t rkey;
        } atomic;
        struct {
            ibv_ah*  ah;
            uint32_t remote_qpn;
            uint32_t remote_qkey;
        } ud;
    } wr;
    union {
        struct {
            uint32_t remote_srqn;
        } xrc;
    } qp_type;
    union {
        struct {
            ibv_mw*  mw;
            uint32_t rkey;
            struct {
                ibv_mr*  mr;
                uint64_t addr;
                uint64_t length;
                unsigned mw_access_flags;
            } bind_info;
        } bind_mw;
        struct {
            void*    hdr;
            uint16_t hdr_sz;
            uint16_t mss;
        } tso;
    };
};

struct ibv_recv_wr {
    uint64_t     wr_id;
    ibv_recv_wr* next;
    ibv_sge*     sg_list;
    int          num_sge;
};

enum { IBV_WC_SEND = 0, IBV_WC_RDMA_WRITE = 1, IBV_WC_RDMA_READ = 2, IBV_WC_RECV = 128, IBV_WC_RECV_RDMA_WITH_IMM = 129 };
enum { IBV_WC_WITH_IMM = 1 << 1 };

struct ibv_wc {
    uint64_t wr_id;
    int      status;
    int      opcode;
    uint32_t vendor_err;
    uint32_t byte_len;
    uint32_t imm_data;
    uint32_t qp_num;
    uint32_t src_qp;
    unsigned wc_flags;
    uint16_t pkey_index;
    uint16_t slid;
    uint8_t  sl;
    uint8_t  dlid_path_bits;
};

struct ibv_context_ops {
    void* compat_query_device;
    void* compat_query_port;
    void* compat_alloc_pd;
    void* compat_dealloc_pd;
    void* compat_reg_mr;
    void* compat_rereg_mr;
    void* compat_dereg_mr;
    ibv_mw* (*alloc_mw)(ibv_pd*, int);
    int (*bind_mw)(ibv_qp*, ibv_mw*, ibv_mw_bind*);
    int (*dealloc_mw)(ibv_mw*);
    void* compat_create_cq;
    int (*poll_cq)(ibv_cq*, int, ibv_wc*);
    int (*req_notify_cq)(ibv_cq*, int);
    void* compat_cq_event;
    void* compat_resize_cq;
    void* compat_destroy_cq;
    void* compat_create_srq;
    void* compat_modify_srq;
    void* compat_query_srq;
    void* compat_destroy_srq;
    int (*post_srq_recv)(ibv_srq*, ibv_recv_wr*, ibv_recv_wr**);
    void* compat_create_qp;
    void* compat_query_qp;
    void* compat_modify_qp;
    void* compat_destroy_qp;
    int (*post_send)(ibv_qp*, ibv_send_wr*, ibv_send_wr**);
    int (*post_recv)(ibv_qp*, ibv_recv_wr*, ibv_recv_wr**);
    void* compat_attach_mcast;
    void* compat_detach_mcast;
    void* compat_async_event;
};

struct ibv_context {
    ibv_device*     device;
    ibv_context_ops ops;
    int             cmd_fd;
    int             async_fd;
    int             num_comp_vectors;
    pthread_mutex_t mutex;
    void*           abi_compat;
};

struct ibv_comp_channel {
    ibv_context* context;
    int          fd;
    int          refcnt;
};

struct ibv_cq {
    ibv_context*      context;
    ibv_comp_channel* channel;
    void*             cq_context;
    uint32_t          handle;
    int               cqe;
    // mutex, cond and event counters follow; not touched here
};

struct ibv_qp {
    ibv_context* context;
    void*        qp_context;
    ibv_pd*      pd;
    ibv_cq*      send_cq;
    ibv_cq*      recv_cq;
    ibv_srq*     srq;
    uint32_t     handle;
    uint32_t     qp_num;
    int          state;
    int          qp_type;
    // mutex, cond and event counter follow; not touched here
};

}  // extern "C"
