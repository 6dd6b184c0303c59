// Starts a communicator's device path: peer windows when every rank can share them, else the
// staged path, the same choice on every rank.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "device/window_path.h"

namespace hx {

std::unique_ptr<DevicePath> make_staged_path(hxcclComm* c);

std::unique_ptr<DevicePath> start_device_path(hxcclComm* c, hxcclResult_t* rc, std::string* why) {
  *rc = hxcclSuccess;
  const char* force = std::getenv("HXCCL_DEVICE_TRANSPORT");
  int staged = force && std::strcmp(force, "staged") == 0 ? 1 : 0;
  if (c->chan->max_int(&staged) != hxcclSuccess) {  // one rank's wish binds all
    *rc = hxcclSystemError;
    *why = "device path setup failed: " + c->chan->error;
    return nullptr;
  }
  std::string window_why = "HXCCL_DEVICE_TRANSPORT=staged";
  if (!staged) {
    auto w = std::make_unique<WindowPath>(c);
    const hxcclResult_t r = w->init();
    if (r == hxcclSuccess) return w;
    window_why = w->error;
  }
  if (std::getenv("HXCCL_DEBUG") && c->rank == 0)
    std::fprintf(stderr, "hxccl: device transport: staged through host memory (%s)\n", window_why.c_str());
  return make_staged_path(c);
}

}  // namespace hx
