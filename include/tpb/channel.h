// Abstract channel interfaces: a channel moves tensor bytes between two endpoints and may use
// transport connections (handed over by the pipe) for its control traffic. Counterpart of
// tensorpipe/channel/{context,channel}.h. The k-th send on one endpoint is matched with the k-th
// recv on the other; callbacks may complete out of order (the pipe re-orders them).
//
// Beyond the reference: sendBatch/recvBatch hand a channel all tensors of one message that it
// carries, so that a device channel can move them with ONE fused kernel launch and one control
// frame; the default implementation just loops over send/recv.
#pragma once

#include <cstddef>
#include <functional>
#include <memory>
#include <optional>
#include <string>
#include <unordered_map>
#include <vector>

#include <tpb/buffer.h>
#include <tpb/device.h>
#include <tpb/error.h>
#include <tpb/message.h>
#include <tpb/transport.h>

namespace tpb {
namespace channel {

enum class Endpoint : bool { kConnect, kListen };

using TSendCallback = std::function<void(const Error&)>;
using TRecvCallback = std::function<void(const Error&)>;

struct SendItem {
  Buffer buffer;
  size_t length = 0;                 // packed bytes in the source dtype
  DType dtype = DType::kBytes;
  std::optional<StridedView> view;   // non-contiguous source
  Device targetDevice;               // where the peer will put it (known to the pipe)
  TSendCallback callback;
};

struct RecvItem {
  Buffer buffer;
  size_t length = 0;                 // packed bytes in the SOURCE dtype (what the descriptor says)
  std::optional<DType> castTo;       // convert while moving; buffer holds the converted size
  DType srcDtype = DType::kBytes;    // element type of the incoming data (needed with castTo)
  Device sourceDevice;
  TRecvCallback callback;
};

class Channel {
 public:
  virtual void send(Buffer buffer, size_t length, TSendCallback callback) = 0;
  virtual void recv(Buffer buffer, size_t length, TRecvCallback callback) = 0;

  virtual void sendBatch(std::vector<SendItem> items) {
    for (auto& it : items) {
      if (it.view.has_value()) {
        it.callback(TPB_CREATE_ERROR(LogicError, "this channel cannot send strided views"));
        continue;
      }
      send(it.buffer, it.length, std::move(it.callback));
    }
  }
  virtual void recvBatch(std::vector<RecvItem> items) {
    for (auto& it : items) {
      if (it.castTo.has_value()) {
        it.callback(TPB_CREATE_ERROR(LogicError, "this channel cannot cast while receiving"));
        continue;
      }
      recv(it.buffer, it.length, std::move(it.callback));
    }
  }
  // True if sendBatch/recvBatch understand StridedView and castTo.
  virtual bool supportsLayouts() const { return false; }

  virtual void setId(std::string id) = 0;
  virtual void close() = 0;
  virtual ~Channel() = default;
};

class Context {
 public:
  virtual bool isViable() const = 0;
  virtual size_t numConnectionsNeeded() const { return 1; }
  // One opaque descriptor per local device this channel can serve.
  virtual const std::unordered_map<Device, std::string>& deviceDescriptors() const = 0;
  virtual bool canCommunicateWithRemote(
      const std::string& localDeviceDescriptor,
      const std::string& remoteDeviceDescriptor) const {
    return localDeviceDescriptor == remoteDeviceDescriptor;
  }
  virtual std::shared_ptr<Channel> createChannel(
      std::vector<std::shared_ptr<transport::Connection>> connections, Endpoint endpoint) = 0;
  virtual void setId(std::string id) = 0;
  virtual void close() = 0;
  virtual void join() = 0;
  virtual ~Context() = default;
};

// ---- factories ------------------------------------------------------------------------------
namespace basic {
std::shared_ptr<Context> create();
}
namespace xth {
std::shared_ptr<Context> create();
}
namespace cma {
std::shared_ptr<Context> create();
}
namespace mpt {
std::shared_ptr<Context> create(
    std::vector<std::shared_ptr<transport::Context>> contexts,
    std::vector<std::shared_ptr<transport::Listener>> listeners);
}
namespace cuda_basic {
// Universal fallback for CUDA tensors: stages through pinned host memory with pack/unpack
// kernels and moves the staged bytes with any CPU channel.
std::shared_ptr<Context> create(std::shared_ptr<Context> cpuContext);
}
namespace cuda_p2p {
// Every field can be overridden from the environment when the channel is created:
// TPB_CUDA_P2P_EAGER_THRESHOLD, _INBOX_BYTES, _MAX_CTAS, _WAIT_KERNEL (0/1), _FUSED_WAIT (0/1),
// _WAIT_TIMEOUT_MS, _BULK (0/1), _CLOSE_TIMEOUT_MS, _HOST_COPY_MIN_BYTES, _HOST_PIECE_BYTES, _SEND_ORDER_MIN_BYTES.
struct Options {
  size_t eagerThreshold = 64 * 1024;     // batches up to this many bytes go through the inbox: one
                                          // control hop less (lower latency), one small kernel more on
                                          // the receiver (which is why larger batches do not)
  size_t inboxBytes = 16u << 20;         // per-peer inbox ring in device memory
  int maxCtas = 0;                        // 0 = one persistent CTA per SM, shared between the
                                          // channels that are sending from that GPU at the moment
  bool waitWithKernel = false;            // true: bounded wait kernel; false: stream memory op
  bool fuseWaitIntoUnpack = true;         // small messages from ANOTHER GPU: the unpack kernel waits itself
  uint64_t waitTimeoutNs = 2'000'000'000ull;  // bound of every device-side wait
  bool useBulkCopy = true;                // TMA bulk pipeline for aligned contiguous data
  uint64_t closeTimeoutMs = 3000;         // how long a closing end waits for the peer's goodbye
  size_t hostCopyMinBytes = 8u << 20;    // a tensor in pinned host memory of at least this size is
                                          // brought in by the copy engine (straight into a receiver
                                          // on the same GPU; in pieces forwarded by the kernel to
                                          // another GPU); smaller ones the kernel reads in place;
                                          // 0: always the kernel
  size_t hostPieceBytes = 32u << 20;     // size of those pieces (two slots of device memory per
                                          // sending GPU, allocated on first use)
  size_t sendOrderMinBytes = 8u << 20;   // a batch of at least this many bytes (all of it on one stream)
                                          // takes its place in the sender's stream when send() is called,
                                          // not when the receiver's buffers become known: an event is
                                          // recorded on that stream by the calling thread, the push runs on
                                          // a stream of the channel's own (highest priority) behind that
                                          // event, and the sender's stream is made to wait for the push at
                                          // the point it has reached by then. Work that the user queues
                                          // between send() and the receiver's answer (the next micro-batch
                                          // of a pipeline) therefore neither delays the push nor is delayed
                                          // by it. The send callback fires as for any other batch. Smaller
                                          // batches are launched on the sender's stream itself, where the
                                          // four extra driver calls would show, and so is a batch that
                                          // stays on its GPU within one process (a local copy). 0: never
  // Host-side fault injection for tests: the N-th push of a channel (counting from 0) is announced
  // to the receiver but not launched, so that the receiver's bounded wait runs out. -1: never.
  int faultSkipLaunch = -1;
};
// The device-to-device channel: a persistent sm_100a kernel on the sender pushes straight into
// the receiver's memory (same process: raw pointers; other process: IPC-mapped) and publishes a
// release-ordered flag. Replaces both cuda_xth and cuda_ipc of the reference.
std::shared_ptr<Context> create(Options options = Options());
// The options after the environment overrides (what create() will use).
Options applyEnvironment(Options options);
// Tensors this process received through a staging buffer because CUDA IPC could not export the
// user's buffer (memory from cudaMallocAsync pools or virtual-memory allocations): a statistic.
uint64_t stagedReceives();
}  // namespace cuda_p2p
namespace cuda_xth {
inline std::shared_ptr<Context> create() { return cuda_p2p::create(); }
}
namespace cuda_ipc {
inline std::shared_ptr<Context> create() { return cuda_p2p::create(); }
}
namespace cuda_gdr {
// GPU memory to GPU memory across hosts through the NICs (GPUDirect RDMA writes into the
// receiver's registered buffer). Needs libibverbs, a NIC and the GPU peer-memory kernel module;
// reports a non-viable context where any of them is missing.
std::shared_ptr<Context> create();
}

}  // namespace channel
}  // namespace tpb
