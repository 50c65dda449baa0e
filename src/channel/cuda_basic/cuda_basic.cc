// cuda_basic: the universal fallback for tensors that touch a GPU (cuda<->cuda without peer
// access, cpu<->cuda), staged through pinned host memory and carried by any CPU channel.
//
// Same role and negotiation as the reference's channel (tensorpipe/channel/cuda_basic/
// context_impl.cc:27-128: wraps a CPU channel, never serves cpu->cpu, descriptor = {device type,
// inner descriptor}) with a different data path. The reference issues one cudaMemcpyAsync plus
// one cudaStreamAddCallback per 1 MiB chunk (channel_impl.cc:58-71,117-229). Here:
//
//   stage out  one kernel launch packs as many 2 MiB pieces as there are free pinned slots, of
//              as many tensors of the message as that covers, straight into mapped pinned memory:
//              contiguous bytes, or the packed form of a 2-D strided view (any element range of
//              it), and publishes one host-visible flag with a system-scope release store; a
//              poller thread notices the flag and hands the slots to the CPU channel in order.
//   stage in   the CPU channel fills pinned slots; one kernel launch moves every slot that has
//              arrived since the last launch into its tensor, converting the element type on the
//              way when the receiver asked for that; the slots return to the pool when an event
//              recorded behind the kernel has fired.
//
// Both ends cut every tensor into the same pieces (2 MiB of packed source bytes) and feed the
// inner channel strictly in piece order, because the inner channel matches its k-th send with
// the peer's k-th recv. Views and conversions never change the pieces: a view is packed by the
// sender, a conversion is applied by the receiver, so neither end needs to know what the other
// does and nothing but tensor bytes crosses the inner channel.
#include <atomic>
#include <cstring>
#include <deque>
#include <map>
#include <set>

#include <tpb/channel.h>

#include "channel/nonviable.h"
#include "common/allocator.h"
#include "common/cuda.h"
#include "common/defs.h"
#include "common/loop.h"
#include "common/nop.h"
#include "common/poller.h"
#include "common/trace.h"
#include "kernels/push.h"

namespace tpb {
namespace channel {
namespace cuda_basic {

namespace {

constexpr size_t kPieceBytes = 2u << 20;
constexpr size_t kSlotsPerDirection = 16;
constexpr const char* kInnerPrefix = "tpbcb1:";

struct DeviceDescriptor {
  std::string deviceType;
  std::string cpuDescriptor;
  TPB_NOP_STRUCTURE(DeviceDescriptor, deviceType, cpuDescriptor)
};

// Pinned, mapped staging slots of one direction, allocated on first use and handed out in
// request order by the chunk pool.
struct Slots {
  uint8_t* base = nullptr;
  volatile uint32_t* flags = nullptr;  // one host-visible word per slot
  std::unique_ptr<Allocator> pool;
  bool ensure() {
    if (base) return true;
    void* p = nullptr;
    if (cudaHostAlloc(&p, kPieceBytes * kSlotsPerDirection + 4096, cudaHostAllocPortable | cudaHostAllocMapped) !=
        cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    base = static_cast<uint8_t*>(p);
    flags = reinterpret_cast<volatile uint32_t*>(base + kPieceBytes * kSlotsPerDirection);
    for (size_t i = 0; i < kSlotsPerDirection; ++i) flags[i] = 0;
    pool = std::make_unique<Allocator>(base, kSlotsPerDirection, kPieceBytes);
    return true;
  }
  size_t indexOf(const uint8_t* slot) const { return static_cast<size_t>(slot - base) / kPieceBytes; }
  ~Slots() {
    pool.reset();
    if (base) cudaFreeHost(base);
  }
};

// ---- host-side restatements for the rare CPU ends of a layout --------------------------------
uint16_t floatToBf16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7f800000u) == 0x7f800000u && (x & 0x007fffffu)) return static_cast<uint16_t>((x >> 16) | 0x40);
  return static_cast<uint16_t>((x + 0x7fffu + ((x >> 16) & 1)) >> 16);
}
float bf16ToFloat(uint16_t h) {
  uint32_t x = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}
bool hostCastSupported(DType s, DType d) {
  return (s == DType::kF32 && d == DType::kBF16) || (s == DType::kBF16 && d == DType::kF32);
}
void hostCast(const uint8_t* src, DType s, uint8_t* dst, size_t elems) {
  if (s == DType::kF32) {
    for (size_t i = 0; i < elems; ++i) {
      float f;
      std::memcpy(&f, src + i * 4, 4);
      const uint16_t h = floatToBf16(f);
      std::memcpy(dst + i * 2, &h, 2);
    }
  } else {
    for (size_t i = 0; i < elems; ++i) {
      uint16_t h;
      std::memcpy(&h, src + i * 2, 2);
      const float f = bf16ToFloat(h);
      std::memcpy(dst + i * 4, &f, 4);
    }
  }
}
// Packed elements [first, first + count) of a 2-D view over host memory.
void hostGather(const uint8_t* base, const StridedView& v, size_t es, uint64_t first, uint64_t count, uint8_t* out) {
  for (uint64_t i = 0; i < count; ++i) {
    const uint64_t e = first + i;
    const int64_t r = static_cast<int64_t>(e / v.cols), c = static_cast<int64_t>(e % v.cols);
    std::memcpy(out + i * es, base + (r * v.rowStride + c * v.colStride) * static_cast<int64_t>(es), es);
  }
}

// Packed elements [first, first + count) of a 2-D view over device memory, as kernel entries: a
// ragged end of the first row, whole rows, a ragged start of the last row.
void appendViewRange(kernels::PushPlan& plan, const uint8_t* base, const StridedView& v, uint64_t first,
                     uint64_t count, uint8_t* out) {
  const int64_t es = static_cast<int64_t>(dtypeSize(v.dtype));
  auto add = [&](int64_t row, int64_t col, int64_t rows, int64_t cols) {
    kernels::CopyItem c;
    c.src = base + (row * v.rowStride + col * v.colStride) * es;
    c.dst = out;
    c.srcBytes = static_cast<uint64_t>(rows * cols * es);
    c.srcDtype = c.dstDtype = v.dtype;
    c.strided = true;
    c.view = StridedView{v.dtype, rows, cols, v.rowStride, v.colStride};
    kernels::appendToPlan(plan, c, false);
    out += rows * cols * es;
  };
  uint64_t cur = first, end = first + count;
  const uint64_t cols = static_cast<uint64_t>(v.cols);
  if (cur % cols != 0) {
    const uint64_t n = std::min<uint64_t>(cols - cur % cols, end - cur);
    add(static_cast<int64_t>(cur / cols), static_cast<int64_t>(cur % cols), 1, static_cast<int64_t>(n));
    cur += n;
  }
  if (end - cur >= cols) {
    const uint64_t rows = (end - cur) / cols;
    add(static_cast<int64_t>(cur / cols), 0, static_cast<int64_t>(rows), v.cols);
    cur += rows * cols;
  }
  if (cur < end) add(static_cast<int64_t>(cur / cols), 0, 1, static_cast<int64_t>(end - cur));
}

class ContextImpl;

class ChannelImpl final : public Channel, public std::enable_shared_from_this<ChannelImpl> {
 public:
  ChannelImpl(std::shared_ptr<ContextImpl> ctx, std::shared_ptr<Channel> inner) : ctx_(std::move(ctx)), inner_(std::move(inner)) {}
  ~ChannelImpl() override;
  void init();
  void send(Buffer buffer, size_t length, TSendCallback cb) override {
    SendItem it;
    it.buffer = buffer;
    it.length = length;
    it.callback = std::move(cb);
    std::vector<SendItem> v;
    v.push_back(std::move(it));
    sendBatch(std::move(v));
  }
  void recv(Buffer buffer, size_t length, TRecvCallback cb) override {
    RecvItem it;
    it.buffer = buffer;
    it.length = length;
    it.callback = std::move(cb);
    std::vector<RecvItem> v;
    v.push_back(std::move(it));
    recvBatch(std::move(v));
  }
  void sendBatch(std::vector<SendItem> items) override;
  void recvBatch(std::vector<RecvItem> items) override;
  bool supportsLayouts() const override { return true; }
  void setId(std::string id) override { inner_->setId(id + ".cpu"); }
  void close() override;
  void closeFromLoop(const Error& e);

 private:
  // One tensor of a batch.
  struct Op {
    size_t remaining = 0;  // pieces not yet accounted for
    Error error;
    std::function<void(const Error&)> cb;
    bool cuda = false;
    uint8_t* ptr = nullptr;  // host or device address of the tensor
    int device = -1;
    cudaStream_t stream = nullptr;
    // send side
    std::optional<StridedView> view;
    // recv side
    std::optional<DType> castTo;
    DType srcDtype = DType::kBytes;
  };
  // 2 MiB (or less) of one tensor's packed source bytes.
  struct Piece {
    std::shared_ptr<Op> op;
    uint64_t off = 0;  // in packed source bytes
    size_t len = 0;
    Allocator::TChunk slot;
    bool slotRequested = false;
    bool launched = false;                  // send: the pack kernel has been launched
    uint32_t flagIndex = 0, flagValue = 0;  // send: the flag of the launch that packs this piece
  };
  void sendBatchFromLoop(std::vector<SendItem> items);
  void recvBatchFromLoop(std::vector<RecvItem> items);
  void pumpSend();
  void packReady();
  void pumpRecv();
  void unpackArrived();
  void pieceDone(const std::shared_ptr<Op>& op, const Error& e);
  uint32_t* counterFor(int device, cudaStream_t stream);

  std::shared_ptr<ContextImpl> ctx_;
  std::shared_ptr<Channel> inner_;
  Error error_;
  std::deque<Piece> sendQueue_;   // in piece order; front = next to hand to the inner channel
  std::deque<Piece*> toPack_;     // pieces that got a slot and wait for the next pack launch
  std::deque<Piece> recvQueue_;   // pieces whose inner recv has not been issued yet
  std::deque<Piece> arrived_;     // device-bound pieces that sit in their slot, in order
  bool unpackScheduled_ = false;
  Slots sendSlots_, recvSlots_;
  uint32_t nextFlagValue_ = 1;
  std::map<std::pair<int, cudaStream_t>, uint32_t*> counters_;  // one arrive counter per launching stream
};

class ContextImpl final : public Context, public std::enable_shared_from_this<ContextImpl> {
 public:
  explicit ContextImpl(std::shared_ptr<Context> cpu) : cpu_(std::move(cpu)) {
    const auto& inner = cpu_->deviceDescriptors();
    auto it = inner.find(Device(kCpuDeviceType, 0));
    if (it == inner.end()) return;
    const int n = cudaDeviceCountNoThrow();
    if (n == 0) return;
    auto add = [&](const Device& d) {
      // Same structure as the reference's descriptor (tensorpipe/channel/cuda_basic/context_impl.cc:
      // 27-31,64-80) but with a prefixed inner descriptor, so that a reference peer's cuda_basic
      // never matches: the pieces and the control traffic of the two differ.
      DeviceDescriptor dd;
      dd.deviceType = d.type;
      dd.cpuDescriptor = kInnerPrefix + it->second;
      auto bytes = nop::encode(dd);
      descriptors_[d] = std::string(bytes.begin(), bytes.end());
    };
    add(Device(kCpuDeviceType, 0));
    for (int i = 0; i < n; ++i) add(Device(kCudaDeviceType, i));
    viable_ = true;
  }
  bool isViable() const override { return viable_ && cpu_->isViable(); }
  size_t numConnectionsNeeded() const override { return cpu_->numConnectionsNeeded(); }
  const std::unordered_map<Device, std::string>& deviceDescriptors() const override { return descriptors_; }
  bool canCommunicateWithRemote(const std::string& local, const std::string& remote) const override {
    DeviceDescriptor l, r;
    if (!nop::decode(local.data(), local.size(), l) || !nop::decode(remote.data(), remote.size(), r)) return false;
    if (l.deviceType == kCpuDeviceType && r.deviceType == kCpuDeviceType) return false;  // not our job
    const std::string prefix = kInnerPrefix;
    if (l.cpuDescriptor.compare(0, prefix.size(), prefix) != 0 || r.cpuDescriptor.compare(0, prefix.size(), prefix) != 0)
      return false;
    return cpu_->canCommunicateWithRemote(l.cpuDescriptor.substr(prefix.size()), r.cpuDescriptor.substr(prefix.size()));
  }
  std::shared_ptr<Channel> createChannel(std::vector<std::shared_ptr<transport::Connection>> conns, Endpoint ep) override {
    auto inner = cpu_->createChannel(std::move(conns), ep);
    auto ch = std::make_shared<ChannelImpl>(shared_from_this(), std::move(inner));
    ch->init();
    return ch;
  }
  void setId(std::string id) override { cpu_->setId(id + ".cpu"); }
  void close() override {
    loop_.deferToLoop([this, self = shared_from_this()]() {
      if (closed_) return;
      closed_ = true;
      auto chans = channels_;
      for (auto& w : chans)
        if (auto c = w.lock()) c->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
      channels_.clear();
      cpu_->close();
    });
  }
  void join() override {
    close();
    loop_.runInLoop([]() {});
    poller_.stop();
    cpu_->join();
    loop_.runInLoop([]() {});
  }
  OnDemandLoop loop_;
  Poller poller_;  // the completion poller every device channel uses (common/poller.h)
  bool closed_ = false;
  std::set<std::weak_ptr<ChannelImpl>, std::owner_less<std::weak_ptr<ChannelImpl>>> channels_;

 private:
  std::shared_ptr<Context> cpu_;
  bool viable_ = false;
  std::unordered_map<Device, std::string> descriptors_;
};

ChannelImpl::~ChannelImpl() {
  for (auto& c : counters_) {
    try {
      CudaDeviceGuard g(c.first.first);
      cudaFree(c.second);
    } catch (...) {
    }
  }
}

void ChannelImpl::init() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() {
    if (self->ctx_->closed_) return self->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
    self->ctx_->channels_.insert(self);
  });
}

uint32_t* ChannelImpl::counterFor(int device, cudaStream_t stream) {
  auto key = std::make_pair(device, stream);
  auto it = counters_.find(key);
  if (it != counters_.end()) return it->second;
  void* p = nullptr;
  TPB_CUDA_CHECK(cudaMalloc(&p, 256));
  // Zero it for certain before the first kernel that counts on it can run (that kernel goes to
  // the user's stream, which a memset on the default stream would not be ordered with).
  if (!cudaZeroNow(p, 256, device)) throw std::runtime_error("cannot clear the arrive counter");
  counters_[key] = static_cast<uint32_t*>(p);
  return static_cast<uint32_t*>(p);
}

void ChannelImpl::pieceDone(const std::shared_ptr<Op>& op, const Error& e) {
  if (e && !op->error) op->error = e;
  if (--op->remaining == 0) {
    auto cb = std::move(op->cb);
    cb(op->error ? op->error : error_);
  }
}

void ChannelImpl::sendBatch(std::vector<SendItem> items) {
  auto self = shared_from_this();
  auto shared = std::make_shared<std::vector<SendItem>>(std::move(items));
  ctx_->loop_.deferToLoop([self, shared]() { self->sendBatchFromLoop(std::move(*shared)); });
}

void ChannelImpl::recvBatch(std::vector<RecvItem> items) {
  auto self = shared_from_this();
  auto shared = std::make_shared<std::vector<RecvItem>>(std::move(items));
  ctx_->loop_.deferToLoop([self, shared]() { self->recvBatchFromLoop(std::move(*shared)); });
}

void ChannelImpl::sendBatchFromLoop(std::vector<SendItem> items) {
  for (auto& it : items) {
    if (error_) {
      it.callback(error_);
      continue;
    }
    if (it.length == 0) {
      it.callback(Error::kSuccess);
      continue;
    }
    if (it.view && static_cast<uint64_t>(it.view->rows) * it.view->cols * dtypeSize(it.view->dtype) != it.length) {
      it.callback(TPB_CREATE_ERROR(LogicError, "strided view does not match the tensor length"));
      continue;
    }
    auto op = std::make_shared<Op>();
    op->cb = std::move(it.callback);
    op->remaining = (it.length + kPieceBytes - 1) / kPieceBytes;
    op->view = it.view;
    if (it.buffer.isCuda()) {
      const CudaBuffer& b = it.buffer.unwrap<CudaBuffer>();
      op->cuda = true;
      op->ptr = static_cast<uint8_t*>(b.ptr);
      op->device = cudaDeviceForPointerOrHint(b);
      op->stream = static_cast<cudaStream_t>(b.stream);
    } else {
      op->ptr = static_cast<uint8_t*>(it.buffer.unwrap<CpuBuffer>().ptr);
    }
    for (uint64_t off = 0; off < it.length; off += kPieceBytes) {
      Piece p;
      p.op = op;
      p.off = off;
      p.len = std::min<uint64_t>(kPieceBytes, it.length - off);
      sendQueue_.push_back(std::move(p));
    }
  }
  pumpSend();
}

void ChannelImpl::pumpSend() {
  if (error_) return;
  auto self = shared_from_this();
  try {
    // Slots: every device piece asks for one, in order; the pool answers in that order. A piece
    // that has its slot joins the next pack launch.
    for (auto& p : sendQueue_) {
      if (p.slotRequested || !p.op->cuda) continue;
      if (!sendSlots_.ensure()) throw std::runtime_error("cannot allocate pinned staging memory");
      if (sendSlots_.pool->numAvailable() == 0) break;  // the rest ask when slots come back
      p.slotRequested = true;
      Piece* piece = &p;  // a deque keeps element addresses across push_back and pop_front
      sendSlots_.pool->alloc(p.len, [this, piece](const Error& e, Allocator::TChunk chunk) {
        if (e) return;  // the pool only fails when the channel is going away
        piece->slot = std::move(chunk);
        toPack_.push_back(piece);
      });
    }
    if (!toPack_.empty()) packReady();
    // Hand over: the front piece goes to the CPU channel once its bytes are where they must be.
    while (!sendQueue_.empty()) {
      Piece& front = sendQueue_.front();
      if (front.op->cuda) {
        if (!front.launched) break;
        if (static_cast<int32_t>(sendSlots_.flags[front.flagIndex] - front.flagValue) < 0) break;
        std::atomic_thread_fence(std::memory_order_acquire);
        Piece piece = std::move(front);
        sendQueue_.pop_front();
        // The source is reusable once packed: the tensor completes when all its pieces are
        // packed (stream order). The slot lives on until the CPU channel is done with it.
        Allocator::TChunk slot = piece.slot;
        inner_->send(CpuBuffer{slot.get()}, piece.len, [self, slot](const Error& e) mutable {
          self->ctx_->loop_.deferToLoop([self, slot = std::move(slot), e]() mutable {
            slot.reset();  // back to the pool, on the loop
            if (e) return self->closeFromLoop(e);
            self->pumpSend();
          });
        });
        pieceDone(piece.op, Error::kSuccess);
        continue;
      }
      // A host tensor goes as it lies; a view over host memory is packed here first.
      Piece piece = std::move(front);
      sendQueue_.pop_front();
      const uint8_t* from = piece.op->ptr + piece.off;
      auto keep = std::make_shared<std::vector<uint8_t>>();
      if (piece.op->view) {
        const size_t es = dtypeSize(piece.op->view->dtype);
        keep->resize(piece.len);
        hostGather(piece.op->ptr, *piece.op->view, es, piece.off / es, piece.len / es, keep->data());
        from = keep->data();
      }
      auto op = piece.op;
      inner_->send(CpuBuffer{const_cast<uint8_t*>(from)}, piece.len, [self, op, keep](const Error& e) {
        self->ctx_->loop_.deferToLoop([self, op, e]() {
          self->pieceDone(op, e);
          if (e) self->closeFromLoop(e);
        });
      });
    }
  } catch (const std::exception& ex) {
    closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
  }
}

// One launch for every piece that has a slot by now (of one device and stream at a time): the
// pieces of a large tensor, or many small tensors, or both.
void ChannelImpl::packReady() {
  auto self = shared_from_this();
  while (!toPack_.empty()) {
    const int device = toPack_.front()->op->device;
    cudaStream_t stream = toPack_.front()->op->stream;
    trace::Scope traced("cuda_basic.pack", toPack_.size());
    CudaDeviceGuard g(device);
    kernels::PushPlan plan;
    std::vector<Piece*> group;
    while (!toPack_.empty() && toPack_.front()->op->device == device && toPack_.front()->op->stream == stream) {
      Piece* p = toPack_.front();
      toPack_.pop_front();
      uint8_t* out = p->slot.get();
      if (p->op->view) {
        const size_t es = dtypeSize(p->op->view->dtype);
        appendViewRange(plan, p->op->ptr, *p->op->view, p->off / es, p->len / es, out);
      } else {
        kernels::CopyItem item;
        item.src = p->op->ptr + p->off;
        item.dst = out;
        item.srcBytes = p->len;
        kernels::appendToPlan(plan, item, false);
      }
      group.push_back(p);
    }
    const uint32_t flagIndex = static_cast<uint32_t>(sendSlots_.indexOf(group.front()->slot.get()));
    const uint32_t flagValue = nextFlagValue_++;
    uint32_t* flag = const_cast<uint32_t*>(sendSlots_.flags + flagIndex);
    kernels::launchPush(plan, stream, cudaSmCount(device), flag, flagValue, counterFor(device, stream), nullptr);
    for (Piece* p : group) {
      p->launched = true;
      p->flagIndex = flagIndex;
      p->flagValue = flagValue;
    }
    volatile uint32_t* hostFlag = sendSlots_.flags + flagIndex;
    ctx_->poller_.watch([hostFlag, flagValue]() { return static_cast<int32_t>(*hostFlag - flagValue) >= 0; },
                        [self]() { self->ctx_->loop_.deferToLoop([self]() { self->pumpSend(); }); });
  }
}

void ChannelImpl::recvBatchFromLoop(std::vector<RecvItem> items) {
  for (auto& it : items) {
    if (error_) {
      it.callback(error_);
      continue;
    }
    if (it.length == 0) {
      it.callback(Error::kSuccess);
      continue;
    }
    auto op = std::make_shared<Op>();
    op->cb = std::move(it.callback);
    op->remaining = (it.length + kPieceBytes - 1) / kPieceBytes;
    op->castTo = it.castTo;
    op->srcDtype = it.srcDtype;
    if (it.castTo && *it.castTo == it.srcDtype) op->castTo.reset();
    const char* refused = nullptr;
    if (it.buffer.isCuda()) {
      const CudaBuffer& b = it.buffer.unwrap<CudaBuffer>();
      op->cuda = true;
      op->ptr = static_cast<uint8_t*>(b.ptr);
      op->device = cudaDeviceForPointerOrHint(b);
      op->stream = static_cast<cudaStream_t>(b.stream);
      if (op->castTo && !kernels::castSupported(op->srcDtype, *op->castTo))
        refused = "unsupported dtype conversion requested by the receiver";
    } else {
      op->ptr = static_cast<uint8_t*>(it.buffer.unwrap<CpuBuffer>().ptr);
      if (op->castTo && !hostCastSupported(op->srcDtype, *op->castTo))
        refused = "this conversion is not available for a tensor received on the host";
    }
    if (refused) {
      // The peer is sending this tensor already: without a place for it the channel is over.
      const Error why = TPB_CREATE_ERROR(LogicError, refused);
      op->cb(why);
      closeFromLoop(why);
      continue;
    }
    for (uint64_t off = 0; off < it.length; off += kPieceBytes) {
      Piece p;
      p.op = op;
      p.off = off;
      p.len = std::min<uint64_t>(kPieceBytes, it.length - off);
      recvQueue_.push_back(std::move(p));
    }
  }
  pumpRecv();
}

void ChannelImpl::pumpRecv() {
  if (error_) return;
  auto self = shared_from_this();
  try {
    // Strictly in piece order: the inner channel pairs its k-th recv with the peer's k-th send.
    while (!recvQueue_.empty()) {
      Piece& front = recvQueue_.front();
      if (front.op->cuda && !front.slot) {
        if (front.slotRequested) break;  // the pool will call back
        if (!recvSlots_.ensure()) throw std::runtime_error("cannot allocate pinned staging memory");
        front.slotRequested = true;
        Piece* piece = &front;
        auto answeredInline = std::make_shared<bool>(true);
        recvSlots_.pool->alloc(front.len, [this, self, piece, answeredInline](const Error& e, Allocator::TChunk chunk) {
          if (e || error_) return;  // after a close the piece it was meant for is gone
          piece->slot = std::move(chunk);
          if (!*answeredInline) pumpRecv();  // a slot came back later: carry on from here
        });
        *answeredInline = false;
        if (!front.slot) break;
      }
      Piece piece = std::move(front);
      recvQueue_.pop_front();
      auto op = piece.op;
      if (!op->cuda && !op->castTo) {
        inner_->recv(CpuBuffer{op->ptr + piece.off}, piece.len, [self, op](const Error& e) {
          self->ctx_->loop_.deferToLoop([self, op, e]() {
            self->pieceDone(op, e);
            if (e) self->closeFromLoop(e);
          });
        });
        continue;
      }
      if (!op->cuda) {
        // Host tensor with a conversion: receive into a temporary, convert on arrival.
        auto temp = std::make_shared<std::vector<uint8_t>>(piece.len);
        const uint64_t off = piece.off;
        const size_t len = piece.len;
        inner_->recv(CpuBuffer{temp->data()}, len, [self, op, temp, off, len](const Error& e) {
          self->ctx_->loop_.deferToLoop([self, op, temp, off, len, e]() {
            if (!e) {
              const size_t ses = dtypeSize(op->srcDtype), des = dtypeSize(*op->castTo);
              hostCast(temp->data(), op->srcDtype, op->ptr + off / ses * des, len / ses);
            }
            self->pieceDone(op, e);
            if (e) self->closeFromLoop(e);
          });
        });
        continue;
      }
      auto shared = std::make_shared<Piece>(std::move(piece));
      inner_->recv(CpuBuffer{shared->slot.get()}, shared->len, [self, shared](const Error& e) {
        self->ctx_->loop_.deferToLoop([self, shared, e]() {
          if (e || self->error_) {
            shared->slot.reset();
            self->pieceDone(shared->op, e ? e : self->error_);
            if (e) self->closeFromLoop(e);
            return;
          }
          self->arrived_.push_back(std::move(*shared));
          // Everything that arrives in this turn of the loop shares one unpack launch.
          if (!self->unpackScheduled_) {
            self->unpackScheduled_ = true;
            self->ctx_->loop_.deferToLoop([self]() {
              self->unpackScheduled_ = false;
              self->unpackArrived();
            });
          }
        });
      });
    }
  } catch (const std::exception& ex) {
    closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
  }
}

void ChannelImpl::unpackArrived() {
  if (error_) return;
  auto self = shared_from_this();
  try {
    while (!arrived_.empty()) {
      const int device = arrived_.front().op->device;
      cudaStream_t stream = arrived_.front().op->stream;
      trace::Scope traced("cuda_basic.unpack", arrived_.size());
      CudaDeviceGuard g(device);
      kernels::PushPlan plan;
      auto group = std::make_shared<std::vector<Piece>>();
      while (!arrived_.empty() && arrived_.front().op->device == device && arrived_.front().op->stream == stream) {
        Piece p = std::move(arrived_.front());
        arrived_.pop_front();
        kernels::CopyItem item;
        item.src = p.slot.get();
        item.srcBytes = p.len;
        if (p.op->castTo) {
          const size_t ses = dtypeSize(p.op->srcDtype), des = dtypeSize(*p.op->castTo);
          item.dst = p.op->ptr + p.off / ses * des;
          item.srcDtype = p.op->srcDtype;
          item.dstDtype = *p.op->castTo;
        } else {
          item.dst = p.op->ptr + p.off;
        }
        kernels::appendToPlan(plan, item, false);
        group->push_back(std::move(p));
      }
      kernels::launchPush(plan, stream, cudaSmCount(device), nullptr, 0, nullptr, nullptr);
      // The slots are free again once the kernel has read them.
      auto ev = std::make_shared<CudaEvent>(device);
      ev->record(stream);
      ctx_->poller_.watch([ev]() { return ev->query(); },
                          [self, group, ev]() {
                            self->ctx_->loop_.deferToLoop([self, group]() {
                              for (auto& p : *group) p.slot.reset();
                              self->pumpRecv();
                            });
                          });
      for (auto& p : *group) pieceDone(p.op, Error::kSuccess);  // enqueued on the stream = received
    }
  } catch (const std::exception& ex) {
    closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
  }
}

void ChannelImpl::close() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() { self->closeFromLoop(TPB_CREATE_ERROR(ChannelClosedError)); });
}

void ChannelImpl::closeFromLoop(const Error& e) {
  if (error_) return;
  error_ = e;
  inner_->close();
  ctx_->channels_.erase(weak_from_this());
  toPack_.clear();
  auto sends = std::move(sendQueue_);
  auto recvs = std::move(recvQueue_);
  auto arrived = std::move(arrived_);
  sendQueue_.clear();
  recvQueue_.clear();
  arrived_.clear();
  for (auto& p : sends) pieceDone(p.op, error_);
  for (auto& p : recvs) pieceDone(p.op, error_);
  for (auto& p : arrived) pieceDone(p.op, error_);
}

}  // namespace

std::shared_ptr<Context> create(std::shared_ptr<Context> cpuContext) {
  if (!cpuContext || !cpuContext->isViable()) return std::make_shared<NonViableContext>();
  auto ctx = std::make_shared<ContextImpl>(std::move(cpuContext));
  if (!ctx->isViable()) return std::make_shared<NonViableContext>();
  return ctx;
}

}  // namespace cuda_basic
}  // namespace channel
}  // namespace tpb
