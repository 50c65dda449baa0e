// Umbrella header (tensorpipe/tensorpipe.h + tensorpipe_cuda.h counterpart).
#pragma once
#include <tpb/buffer.h>
#include <tpb/channel.h>
#include <tpb/context.h>
#include <tpb/device.h>
#include <tpb/error.h>
#include <tpb/listener.h>
#include <tpb/message.h>
#include <tpb/pipe.h>
#include <tpb/transport.h>
#include <tpb/trace.h>
