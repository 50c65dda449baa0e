// verbs::systemProvider(): real NICs through libibverbs, loaded with dlopen so that nothing links
// against it. The part of the verbs ABI used here is declared below as rdma-core lays it out
// (infiniband/verbs.h): the structures this file reads or fills, the operation table inside
// ibv_context through which the data-path calls (poll, post) go, and the enumerators. Only what is
// touched is declared in full; the tail of a structure this file never reads is left out where
// the library allocates the object.
//
// Role of tensorpipe/common/ibv_lib.h:20-704 and tensorpipe/common/ibv.cc:78-191. Queue pairs are
// reliable-connected on port 1, GID index 0 by default (TPB_IBV_PORT / TPB_IBV_GID_INDEX override).
#include <pthread.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <stdexcept>

#include "common/defs.h"
#include "common/dl.h"
#include "common/verbs.h"

namespace tpb {
namespace verbs {
namespace {

// ---- the ABI ------------------------------------------------------------------------------------
extern "C" {
struct ibv_context;
struct ibv_pd;
struct ibv_cq;
struct ibv_srq;
struct ibv_qp;
struct ibv_mw;
struct ibv_mw_bind;
struct ibv_ah;
struct ibv_comp_channel;

struct ibv_device {
  void* ops_[2];
  int node_type;
  int transport_type;
  char name[64];
  char dev_name[64];
  char dev_path[256];
  char ibdev_path[256];
};

struct ibv_sge {
  uint64_t addr;
  uint32_t length;
  uint32_t lkey;
};

struct ibv_recv_wr {
  uint64_t wr_id;
  ibv_recv_wr* next;
  ibv_sge* sg_list;
  int num_sge;
};

struct ibv_mw_bind_info {
  void* mr;
  uint64_t addr;
  uint64_t length;
  unsigned int mw_access_flags;
};

struct ibv_send_wr {
  uint64_t wr_id;
  ibv_send_wr* next;
  ibv_sge* sg_list;
  int num_sge;
  int opcode;
  unsigned int send_flags;
  uint32_t imm_data;  // big-endian on the wire
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
      ibv_ah* ah;
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
      ibv_mw* mw;
      uint32_t rkey;
      ibv_mw_bind_info bind_info;
    } bind_mw;
    struct {
      void* hdr;
      uint16_t hdr_sz;
      uint16_t mss;
    } tso;
  };
};

struct ibv_wc {
  uint64_t wr_id;
  int status;
  int opcode;
  uint32_t vendor_err;
  uint32_t byte_len;
  uint32_t imm_data;  // big-endian
  uint32_t qp_num;
  uint32_t src_qp;
  unsigned int wc_flags;
  uint16_t pkey_index;
  uint16_t slid;
  uint8_t sl;
  uint8_t dlid_path_bits;
};

struct ibv_context_ops {
  void* compat_query_device;
  void* compat_query_port;
  void* compat_alloc_pd;
  void* compat_dealloc_pd;
  void* compat_reg_mr;
  void* compat_rereg_mr;
  void* compat_dereg_mr;
  void* alloc_mw;
  void* bind_mw;
  void* dealloc_mw;
  void* compat_create_cq;
  int (*poll_cq)(ibv_cq* cq, int num_entries, ibv_wc* wc);
  void* req_notify_cq;
  void* compat_cq_event;
  void* compat_resize_cq;
  void* compat_destroy_cq;
  void* compat_create_srq;
  void* compat_modify_srq;
  void* compat_query_srq;
  void* compat_destroy_srq;
  int (*post_srq_recv)(ibv_srq* srq, ibv_recv_wr* wr, ibv_recv_wr** bad);
  void* compat_create_qp;
  void* compat_query_qp;
  void* compat_modify_qp;
  void* compat_destroy_qp;
  int (*post_send)(ibv_qp* qp, ibv_send_wr* wr, ibv_send_wr** bad);
  void* post_recv;
  void* compat_create_ah;
  void* compat_destroy_ah;
  void* compat_attach_mcast;
  void* compat_detach_mcast;
  void* compat_async_event;
};

struct ibv_context {
  ibv_device* device;
  ibv_context_ops ops;
  // cmd_fd, async_fd, ... follow; never read here.
};

struct ibv_mr {
  ibv_context* context;
  ibv_pd* pd;
  void* addr;
  size_t length;
  uint32_t handle;
  uint32_t lkey;
  uint32_t rkey;
};

// The leading members of the objects the library allocates; the data-path calls reach the
// operation table through `context`.
struct ibv_cq {
  ibv_context* context;
};
struct ibv_srq {
  ibv_context* context;
};
struct ibv_qp {
  ibv_context* context;
  void* qp_context;
  ibv_pd* pd;
  ibv_cq* send_cq;
  ibv_cq* recv_cq;
  ibv_srq* srq;
  uint32_t handle;
  uint32_t qp_num;
};

union ibv_gid {
  uint8_t raw[16];
};

struct ibv_global_route {
  ibv_gid dgid;
  uint32_t flow_label;
  uint8_t sgid_index;
  uint8_t hop_limit;
  uint8_t traffic_class;
};

struct ibv_ah_attr {
  ibv_global_route grh;
  uint16_t dlid;
  uint8_t sl;
  uint8_t src_path_bits;
  uint8_t static_rate;
  uint8_t is_global;
  uint8_t port_num;
};

struct ibv_qp_cap {
  uint32_t max_send_wr;
  uint32_t max_recv_wr;
  uint32_t max_send_sge;
  uint32_t max_recv_sge;
  uint32_t max_inline_data;
};

struct ibv_qp_init_attr {
  void* qp_context;
  ibv_cq* send_cq;
  ibv_cq* recv_cq;
  ibv_srq* srq;
  ibv_qp_cap cap;
  int qp_type;
  int sq_sig_all;
};

struct ibv_srq_attr {
  uint32_t max_wr;
  uint32_t max_sge;
  uint32_t srq_limit;
};

struct ibv_srq_init_attr {
  void* srq_context;
  ibv_srq_attr attr;
};

struct ibv_qp_attr {
  int qp_state;
  int cur_qp_state;
  int path_mtu;
  int path_mig_state;
  uint32_t qkey;
  uint32_t rq_psn;
  uint32_t sq_psn;
  uint32_t dest_qp_num;
  unsigned int qp_access_flags;
  ibv_qp_cap cap;
  ibv_ah_attr ah_attr;
  ibv_ah_attr alt_ah_attr;
  uint16_t pkey_index;
  uint16_t alt_pkey_index;
  uint8_t en_sqd_async_notify;
  uint8_t sq_draining;
  uint8_t max_rd_atomic;
  uint8_t max_dest_rd_atomic;
  uint8_t min_rnr_timer;
  uint8_t port_num;
  uint8_t timeout;
  uint8_t retry_cnt;
  uint8_t rnr_retry;
  uint8_t alt_port_num;
  uint8_t alt_timeout;
  uint32_t rate_limit;
};

struct ibv_port_attr {
  int state;
  int max_mtu;
  int active_mtu;
  int gid_tbl_len;
  uint32_t port_cap_flags;
  uint32_t max_msg_sz;
  uint32_t bad_pkey_cntr;
  uint32_t qkey_viol_cntr;
  uint16_t pkey_tbl_len;
  uint16_t lid;
  uint16_t sm_lid;
  uint8_t lmc;
  uint8_t max_vl_num;
  uint8_t sm_sl;
  uint8_t subnet_timeout;
  uint8_t init_type_reply;
  uint8_t active_width;
  uint8_t active_speed;
  uint8_t phys_state;
  uint8_t link_layer;
  uint8_t flags;
  uint16_t port_cap_flags2;
  uint32_t active_speed_ex;
  uint8_t reserved_[64];  // room for what later versions of the library append
};
}  // extern "C"

enum : int { kQpsReset = 0, kQpsInit = 1, kQpsRtr = 2, kQpsRts = 3, kQpsErr = 6 };
enum : int { kQptRc = 2 };
enum : int { kWrRdmaWriteWithImm = 1, kWrSendWithImm = 3 };
enum : unsigned { kSendSignaled = 2 };
enum : unsigned { kAccessLocalWrite = 1, kAccessRemoteWrite = 2 };
enum : int { kWcSend = 0, kWcRdmaWrite = 1, kWcRecv = 128, kWcRecvRdmaWithImm = 129 };
enum : int {
  kQpState = 1 << 0,
  kQpAccessFlags = 1 << 3,
  kQpPkeyIndex = 1 << 4,
  kQpPort = 1 << 5,
  kQpAv = 1 << 7,
  kQpPathMtu = 1 << 8,
  kQpTimeout = 1 << 9,
  kQpRetryCnt = 1 << 10,
  kQpRnrRetry = 1 << 11,
  kQpRqPsn = 1 << 12,
  kQpMaxQpRdAtomic = 1 << 13,
  kQpMinRnrTimer = 1 << 15,
  kQpSqPsn = 1 << 16,
  kQpMaxDestRdAtomic = 1 << 17,
  kQpDestQpn = 1 << 20,
};

struct Lib {
  bool ok = false;
  std::string why;
  ibv_device** (*get_device_list)(int*) = nullptr;
  void (*free_device_list)(ibv_device**) = nullptr;
  ibv_context* (*open_device)(ibv_device*) = nullptr;
  int (*close_device)(ibv_context*) = nullptr;
  int (*query_port)(ibv_context*, uint8_t, ibv_port_attr*) = nullptr;
  int (*query_gid)(ibv_context*, uint8_t, int, ibv_gid*) = nullptr;
  ibv_pd* (*alloc_pd)(ibv_context*) = nullptr;
  int (*dealloc_pd)(ibv_pd*) = nullptr;
  ibv_mr* (*reg_mr)(ibv_pd*, void*, size_t, int) = nullptr;
  int (*dereg_mr)(ibv_mr*) = nullptr;
  ibv_cq* (*create_cq)(ibv_context*, int, void*, ibv_comp_channel*, int) = nullptr;
  int (*destroy_cq)(ibv_cq*) = nullptr;
  ibv_srq* (*create_srq)(ibv_pd*, ibv_srq_init_attr*) = nullptr;
  int (*destroy_srq)(ibv_srq*) = nullptr;
  ibv_qp* (*create_qp)(ibv_pd*, ibv_qp_init_attr*) = nullptr;
  int (*destroy_qp)(ibv_qp*) = nullptr;
  int (*modify_qp)(ibv_qp*, ibv_qp_attr*, int) = nullptr;
  const char* (*wc_status_str)(int) = nullptr;
  void* handle = nullptr;

  static const Lib& get() {
    static Lib lib = [] {
      Lib l;
      DynamicLibraryHandle dl("libibverbs.so.1");
      if (!dl.loaded()) {
        l.why = dl.error();
        return l;
      }
      const bool all = dl.load(l.get_device_list, {"ibv_get_device_list"}) &&
          dl.load(l.free_device_list, {"ibv_free_device_list"}) && dl.load(l.open_device, {"ibv_open_device"}) &&
          dl.load(l.close_device, {"ibv_close_device"}) && dl.load(l.query_port, {"ibv_query_port"}) &&
          dl.load(l.query_gid, {"ibv_query_gid"}) && dl.load(l.alloc_pd, {"ibv_alloc_pd"}) &&
          dl.load(l.dealloc_pd, {"ibv_dealloc_pd"}) && dl.load(l.reg_mr, {"ibv_reg_mr"}) &&
          dl.load(l.dereg_mr, {"ibv_dereg_mr"}) && dl.load(l.create_cq, {"ibv_create_cq"}) &&
          dl.load(l.destroy_cq, {"ibv_destroy_cq"}) && dl.load(l.create_srq, {"ibv_create_srq"}) &&
          dl.load(l.destroy_srq, {"ibv_destroy_srq"}) && dl.load(l.create_qp, {"ibv_create_qp"}) &&
          dl.load(l.destroy_qp, {"ibv_destroy_qp"}) && dl.load(l.modify_qp, {"ibv_modify_qp"}) &&
          dl.load(l.wc_status_str, {"ibv_wc_status_str"});
      l.handle = dl.release();  // stays mapped: the entry points above are kept
      if (!all) {
        l.why = "libibverbs.so.1 lacks required symbols";
        return l;
      }
      l.ok = true;
      return l;
    }();
    return lib;
  }
};

int envInt(const char* name, int fallback) {
  const char* s = std::getenv(name);
  if (!s || !*s) return fallback;
  return std::atoi(s);
}

uint32_t toBigEndian(uint32_t v) { return __builtin_bswap32(v); }

[[noreturn]] void fail(const std::string& what, int err) {
  throw std::runtime_error(what + ": " + std::strerror(err));
}

struct SysRegion final : MemoryRegion {
  explicit SysRegion(ibv_mr* mr) : mr(mr) {}
  ~SysRegion() override { Lib::get().dereg_mr(mr); }
  uint32_t localKey() const override { return mr->lkey; }
  uint32_t remoteKey() const override { return mr->rkey; }
  ibv_mr* mr;
};

struct SysCq final : CompletionQueue {
  explicit SysCq(ibv_cq* cq) : cq(cq) {}
  ~SysCq() override { Lib::get().destroy_cq(cq); }
  int poll(Completion* out, int max) override {
    constexpr int kBatch = 32;
    ibv_wc wcs[kBatch];
    if (max > kBatch) max = kBatch;
    const int n = cq->context->ops.poll_cq(cq, max, wcs);
    if (n < 0) throw std::runtime_error("polling the completion queue failed");
    for (int i = 0; i < n; ++i) {
      const ibv_wc& wc = wcs[i];
      Completion& c = out[i];
      c = Completion();
      c.id = wc.wr_id;
      c.ok = wc.status == 0;
      if (!c.ok) c.error = Lib::get().wc_status_str(wc.status);
      c.queuePair = wc.qp_num;
      c.byteLength = wc.byte_len;
      c.immediate = toBigEndian(wc.imm_data);
      // A failed completion carries no trustworthy opcode; the poster tells the kinds apart by id.
      switch (wc.opcode) {
        case kWcRdmaWrite: c.work = Work::kWrite; break;
        case kWcSend: c.work = Work::kSend; break;
        case kWcRecvRdmaWithImm: c.work = Work::kWriteArrived; break;
        case kWcRecv: c.work = Work::kSendArrived; break;
        default: c.work = Work::kWrite; break;
      }
    }
    return n;
  }
  ibv_cq* cq;
};

struct SysSrq final : SharedReceiveQueue {
  explicit SysSrq(ibv_srq* srq) : srq(srq) {}
  ~SysSrq() override { Lib::get().destroy_srq(srq); }
  void postReceive(uint64_t id, ReceiveBuffer buffer) override {
    ibv_sge sge{reinterpret_cast<uint64_t>(buffer.ptr), buffer.length, buffer.localKey};
    ibv_recv_wr wr{};
    wr.wr_id = id;
    wr.sg_list = buffer.length ? &sge : nullptr;
    wr.num_sge = buffer.length ? 1 : 0;
    ibv_recv_wr* bad = nullptr;
    const int rc = srq->context->ops.post_srq_recv(srq, &wr, &bad);
    if (rc != 0) fail("posting a receive", rc);
  }
  ibv_srq* srq;
};

struct SysQp final : QueuePair {
  SysQp(ibv_qp* qp, uint8_t port, uint8_t gidIndex) : qp(qp), port(port), gidIndex(gidIndex) {}
  ~SysQp() override { Lib::get().destroy_qp(qp); }
  uint32_t number() const override { return qp->qp_num; }
  void toInit() override {
    ibv_qp_attr a{};
    a.qp_state = kQpsInit;
    a.pkey_index = 0;
    a.port_num = port;
    a.qp_access_flags = kAccessLocalWrite | kAccessRemoteWrite;
    modify(a, kQpState | kQpPkeyIndex | kQpPort | kQpAccessFlags, "INIT");
  }
  void toReadyToReceive(const Address& remote) override {
    ibv_qp_attr a{};
    a.qp_state = kQpsRtr;
    a.path_mtu = remote.mtu;
    a.dest_qp_num = remote.queuePair;
    a.rq_psn = remote.packetSequence;
    a.max_dest_rd_atomic = 1;
    a.min_rnr_timer = 20;  // 10.24 ms between receiver-not-ready retries
    a.ah_attr.dlid = static_cast<uint16_t>(remote.localId);
    a.ah_attr.port_num = port;
    // Without a local id the port is Ethernet (RoCE): route by global id.
    if (remote.localId == 0) {
      a.ah_attr.is_global = 1;
      std::memcpy(a.ah_attr.grh.dgid.raw, remote.gid.data(), 16);
      a.ah_attr.grh.sgid_index = gidIndex;
      a.ah_attr.grh.hop_limit = 1;
    }
    modify(a, kQpState | kQpAv | kQpPathMtu | kQpDestQpn | kQpRqPsn | kQpMaxDestRdAtomic | kQpMinRnrTimer,
           "ready-to-receive");
  }
  void toReadyToSend(uint32_t ownPacketSequence) override {
    ibv_qp_attr a{};
    a.qp_state = kQpsRts;
    a.sq_psn = ownPacketSequence;
    a.timeout = 14;    // 4.096 us * 2^14 = 67 ms per transport retry
    a.retry_cnt = 7;
    a.rnr_retry = 7;   // retry for ever while the receiver has nothing posted
    a.max_rd_atomic = 1;
    modify(a, kQpState | kQpSqPsn | kQpTimeout | kQpRetryCnt | kQpRnrRetry | kQpMaxQpRdAtomic, "ready-to-send");
  }
  void toError() override {
    ibv_qp_attr a{};
    a.qp_state = kQpsErr;
    Lib::get().modify_qp(qp, &a, kQpState);  // best effort: already in error is fine
  }
  void postWriteWithImmediate(uint64_t id, const void* local, uint32_t length, uint32_t localKey, uint64_t remoteAddress,
                              uint32_t remoteKey, uint32_t immediate) override {
    ibv_sge sge{reinterpret_cast<uint64_t>(local), length, localKey};
    ibv_send_wr wr{};
    wr.wr_id = id;
    wr.sg_list = &sge;
    wr.num_sge = 1;
    wr.opcode = kWrRdmaWriteWithImm;
    wr.send_flags = kSendSignaled;
    wr.imm_data = toBigEndian(immediate);
    wr.wr.rdma.remote_addr = remoteAddress;
    wr.wr.rdma.rkey = remoteKey;
    post(wr, "posting an RDMA write");
  }
  void postSendWithImmediate(uint64_t id, const void* local, uint32_t length, uint32_t localKey, uint32_t immediate) override {
    ibv_sge sge{reinterpret_cast<uint64_t>(local), length, localKey};
    ibv_send_wr wr{};
    wr.wr_id = id;
    wr.sg_list = length ? &sge : nullptr;
    wr.num_sge = length ? 1 : 0;
    wr.opcode = kWrSendWithImm;
    wr.send_flags = kSendSignaled;
    wr.imm_data = toBigEndian(immediate);
    post(wr, "posting a send");
  }
  void modify(ibv_qp_attr& a, int mask, const char* to) {
    const int rc = Lib::get().modify_qp(qp, &a, mask);
    if (rc != 0) fail(std::string("moving a queue pair to ") + to, rc);
  }
  void post(ibv_send_wr& wr, const char* what) {
    ibv_send_wr* bad = nullptr;
    const int rc = qp->context->ops.post_send(qp, &wr, &bad);
    if (rc != 0) fail(what, rc);
  }
  ibv_qp* qp;
  uint8_t port, gidIndex;
};

struct SysDevice final : Device {
  SysDevice(ibv_context* ctx, std::string name, std::string pci) : ctx(ctx), name_(std::move(name)), pci_(std::move(pci)) {
    const Lib& lib = Lib::get();
    port = static_cast<uint8_t>(envInt("TPB_IBV_PORT", 1));
    gidIndex = static_cast<uint8_t>(envInt("TPB_IBV_GID_INDEX", 0));
    pd = lib.alloc_pd(ctx);
    if (!pd) {
      lib.close_device(ctx);
      throw std::runtime_error("allocating a protection domain on " + name_ + " failed");
    }
    ibv_port_attr pa{};
    if (lib.query_port(ctx, port, &pa) != 0) {
      lib.dealloc_pd(pd);
      lib.close_device(ctx);
      throw std::runtime_error("querying port " + std::to_string(port) + " of " + name_ + " failed");
    }
    address_.localId = pa.lid;
    address_.mtu = static_cast<uint8_t>(pa.active_mtu);
    maxMessage_ = pa.max_msg_sz ? pa.max_msg_sz : (1u << 30);
    ibv_gid gid{};
    if (lib.query_gid(ctx, port, gidIndex, &gid) == 0) std::memcpy(address_.gid.data(), gid.raw, 16);
  }
  ~SysDevice() override {
    Lib::get().dealloc_pd(pd);
    Lib::get().close_device(ctx);
  }
  const std::string& name() const override { return name_; }
  const std::string& pciPath() const override { return pci_; }
  Address portAddress() const override { return address_; }
  uint32_t maxMessageBytes() const override { return maxMessage_; }
  std::unique_ptr<MemoryRegion> registerMemory(void* ptr, size_t length) override {
    ibv_mr* mr = Lib::get().reg_mr(pd, ptr, length, kAccessLocalWrite | kAccessRemoteWrite);
    if (!mr) fail("registering memory with " + name_, errno);
    return std::make_unique<SysRegion>(mr);
  }
  std::unique_ptr<CompletionQueue> createCompletionQueue(int entries) override {
    ibv_cq* cq = Lib::get().create_cq(ctx, entries, nullptr, nullptr, 0);
    if (!cq) fail("creating a completion queue on " + name_, errno);
    return std::make_unique<SysCq>(cq);
  }
  std::unique_ptr<SharedReceiveQueue> createSharedReceiveQueue(int entries) override {
    ibv_srq_init_attr a{};
    a.attr.max_wr = static_cast<uint32_t>(entries);
    a.attr.max_sge = 1;
    ibv_srq* srq = Lib::get().create_srq(pd, &a);
    if (!srq) fail("creating a shared receive queue on " + name_, errno);
    return std::make_unique<SysSrq>(srq);
  }
  std::unique_ptr<QueuePair> createQueuePair(CompletionQueue& cq, SharedReceiveQueue& srq, int sendEntries) override {
    ibv_qp_init_attr a{};
    a.send_cq = static_cast<SysCq&>(cq).cq;
    a.recv_cq = static_cast<SysCq&>(cq).cq;
    a.srq = static_cast<SysSrq&>(srq).srq;
    a.cap.max_send_wr = static_cast<uint32_t>(sendEntries);
    a.cap.max_send_sge = 1;
    a.qp_type = kQptRc;
    a.sq_sig_all = 1;
    ibv_qp* qp = Lib::get().create_qp(pd, &a);
    if (!qp) fail("creating a queue pair on " + name_, errno);
    return std::make_unique<SysQp>(qp, port, gidIndex);
  }
  ibv_context* ctx;
  ibv_pd* pd = nullptr;
  std::string name_, pci_;
  Address address_;
  uint32_t maxMessage_ = 1u << 30;
  uint8_t port = 1, gidIndex = 0;
};

struct SysProvider final : Provider {
  std::vector<std::string> deviceNames() override {
    std::vector<std::string> names;
    const Lib& lib = Lib::get();
    if (!lib.ok) return names;
    int n = 0;
    ibv_device** list = lib.get_device_list(&n);
    if (!list) return names;
    for (int i = 0; i < n; ++i) names.emplace_back(list[i]->name);
    lib.free_device_list(list);
    return names;
  }
  std::unique_ptr<Device> open(const std::string& name) override {
    const Lib& lib = Lib::get();
    if (!lib.ok) throw std::runtime_error("libibverbs is not available: " + lib.why);
    int n = 0;
    ibv_device** list = lib.get_device_list(&n);
    if (!list) throw std::runtime_error("listing InfiniBand devices failed");
    std::unique_ptr<Device> dev;
    std::string why = "no InfiniBand device named " + name;
    for (int i = 0; i < n && !dev; ++i) {
      if (name != list[i]->name) continue;
      ibv_context* ctx = lib.open_device(list[i]);
      if (!ctx) {
        why = "opening " + name + " failed";
        break;
      }
      // The device's place in the PCI tree: /sys/class/infiniband/<name>/device resolved.
      std::string pci;
      {
        const std::string link = std::string(list[i]->ibdev_path) + "/device";
        char* real = ::realpath(link.c_str(), nullptr);
        if (real) {
          pci = real;
          std::free(real);
        }
      }
      try {
        dev = std::make_unique<SysDevice>(ctx, name, pci);
      } catch (const std::exception& ex) {
        why = ex.what();
      }
    }
    lib.free_device_list(list);
    if (!dev) throw std::runtime_error(why);
    return dev;
  }
  std::string whyUnavailable() const override {
    const Lib& lib = Lib::get();
    if (!lib.ok) return lib.why;
    return "no InfiniBand device";
  }
};

}  // namespace

std::shared_ptr<Provider> systemProvider() {
  static std::shared_ptr<Provider> p = std::make_shared<SysProvider>();
  return p;
}

}  // namespace verbs
}  // namespace tpb
