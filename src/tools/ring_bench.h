// Benchmark engine shared by the command-line benchmark, the Python bindings and bench.py.
// Every rank owns a sending context (dials the next rank) and a receiving context (listens for
// the previous rank); with one rank the two contexts talk to each other in-process on one GPU.
// Measures what the reference's benchmark_pipe measures (tensorpipe/benchmark/benchmark_pipe.cc:
// a full Pipe write -> readDescriptor -> read per iteration) but timed on the device.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace tpb {
namespace tools {

struct RingBenchOptions {
  int device = 0;
  bool useShm = true;         // register the shm transport (control traffic) next to TCP
  bool useBulkCopy = true;
  bool waitWithKernel = false;
  size_t eagerThreshold = 64 * 1024;
  int maxCtas = 0;
  size_t maxBytes = 1ull << 30;  // largest tensor that will be sent (buffers are sized for it)
  std::string channel = "cuda_p2p";  // or "cuda_basic"
};

struct PhaseResult {
  double deviceMs = 0;     // CUDA-event time from phase start to the last receive, this rank
  double hostMs = 0;       // wall clock of the same region
  uint64_t mismatches = 0; // bytes that differ from the expected pattern (when verifying)
  uint64_t kernelLaunches = 0;
};

class RingBench {
 public:
  explicit RingBench(RingBenchOptions opts);
  ~RingBench();

  // URL of this rank's receiving listener; give it to the previous rank.
  std::string listenUrl() const;
  // Dial the next rank's listener and accept the previous rank's pipe. Blocks until both exist.
  void connect(const std::string& nextUrl);

  // Stream `steps` messages of one `bytes`-sized tensor to the next rank while receiving the same
  // from the previous one, keeping up to `depth` writes in flight. Every rank must call this
  // with the same arguments.
  PhaseResult runStream(size_t bytes, int steps, int depth, bool verify);

  // One token travels around the ring `laps` times (with one rank: out and back in-process).
  // Returns per-hop latencies in microseconds as seen by this rank (host clock around
  // write -> data visible on the device), one sample per lap. Rank 0 starts the token.
  std::vector<double> runLatency(size_t bytes, int laps, int rank, int world);

  // 64-tensor mixed message (fp32/bf16/int64, a quarter transposed views of 8 to 4096 columns,
  // half of the fp32 tensors cast to bf16 by the receiver), `steps` times. Returns the bytes
  // delivered per step. With `verify` one message is sent from a seeded source and every delivered
  // element is compared with a CPU restatement (result in PhaseResult::mismatches; nothing is timed).
  PhaseResult runMixed(int steps, uint64_t seed, uint64_t* bytesPerStep, bool verify);

  // The ring end to end through the public C++ API (Pipe::write / readDescriptor / read), one
  // message at a time: every step's tensor starts in pinned host memory, which is what is handed
  // to Pipe::write (as a tensor of this rank's GPU), and the step ends when four bytes of the
  // received tensor have been copied back to pinned host memory and both streams are idle.
  // `prepare` allocates and fills the pinned source with a seeded pattern (untimed); `steps` timed
  // steps follow; with `verify` the last received tensor is compared with the pattern on the
  // device afterwards. hostMs is the wall clock of the steps.
  PhaseResult runEndToEnd(size_t bytes, int steps, bool verify);

  // All-pairs mode: dial every other rank's listener ("url|device" per rank, own entry ignored) and
  // accept everybody's pipe; then every rank sends the mixed message to every other rank at once.
  void connectMesh(const std::vector<std::string>& urls, int rank);
  PhaseResult runMixedMesh(int steps, uint64_t seed, uint64_t* bytesPerMessage);

 private:
  struct Impl;
  std::unique_ptr<Impl> impl_;
};

}  // namespace tools
}  // namespace tpb
