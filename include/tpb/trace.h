// Timeline tracing (not in the reference, whose substitutes are verbose logs and the state-machine
// dump tool). Off by default; when on, pipes, channels and kernel launches record begin/end and
// instant events into a lock-free ring that dumps as a chrome://tracing JSON file. The same
// ranges are emitted through NVTX for tools that inject an NVTX backend.
//
//   TPB_TRACE=/path/trace.json    trace from start-up, dump at exit
#pragma once

#include <cstdint>
#include <string>

namespace tpb {

// Starts recording; `path` is where traceDump() writes by default.
void traceEnable(const std::string& path);
void traceDisable();
// Writes the most recent events (at most 65536). False if tracing never started or on I/O error.
bool traceDump(const std::string& path = "");
// Events recorded so far, including those the ring has already overwritten.
uint64_t traceEventCount();

}  // namespace tpb
