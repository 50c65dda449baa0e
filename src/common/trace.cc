#include "common/trace.h"

#include <tpb/trace.h>

namespace tpb {

void traceEnable(const std::string& path) { trace::Tracer::get().enable(path); }
void traceDisable() { trace::Tracer::get().disable(); }
bool traceDump(const std::string& path) { return trace::Tracer::get().dump(path); }
uint64_t traceEventCount() { return trace::Tracer::get().count(); }

}  // namespace tpb
