// hxcclGroupStart / hxcclGroupEnd bookkeeping (reference behaviour: src/group.cc:22-110).
#pragma once
#include "core/comm.h"

namespace hx {

// Runs `work` now, or queues it until the outermost hxcclGroupEnd.
hxcclResult_t dispatch(hxcclComm* c, Deferred work);
// One Send or Recv: runs now (alone), or joins the open group.
hxcclResult_t submit_p2p(hxcclComm* c, Path path, bool is_send, int peer, void* buf,
                         size_t bytes, void* stream);

}  // namespace hx
