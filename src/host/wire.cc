#include "wire.h"

namespace hx {

bool HostWire::injected() {
  if (fail_after < 0) return false;
  if (fail_after-- > 0) return false;
  error = "injected transport failure";
  return true;
}

hxcclResult_t HostWire::post_send(int to, const void* buf, size_t bytes, int tag, bool fragment) {
  if (injected()) return hxcclSystemError;
  open_.push_back(ch_->post_send(to, tag, buf, bytes));
  bytes_sent += bytes;
  if (!fragment) ++msgs_sent;
  return hxcclSuccess;
}

hxcclResult_t HostWire::post_recv(int from, void* buf, size_t bytes, int tag) {
  open_.push_back(ch_->post_recv(from, tag, buf, bytes));
  return hxcclSuccess;
}

hxcclResult_t HostWire::step(bool* done) {
  for (size_t i = 0; i < open_.size();) {
    bool fin = false;
    const hxcclResult_t r = ch_->poll_ticket(open_[i], &fin);
    if (!fin) {
      ++i;
      continue;
    }
    if (r != hxcclSuccess && first_ == hxcclSuccess) {
      first_ = r;
      first_why_ = ch_->error;
    }
    open_[i] = open_.back();
    open_.pop_back();
  }
  *done = open_.empty();
  if (!*done) return hxcclSuccess;
  const hxcclResult_t r = first_;
  if (r != hxcclSuccess) error = first_why_;
  first_ = hxcclSuccess;
  first_why_.clear();
  return r;
}

hxcclResult_t HostWire::finish_all() {
  for (int t : open_) {
    const hxcclResult_t r = ch_->wait_ticket(t);
    if (r != hxcclSuccess && first_ == hxcclSuccess) {
      first_ = r;
      first_why_ = ch_->error;
    }
  }
  open_.clear();
  const hxcclResult_t r = first_;
  if (r != hxcclSuccess) error = first_why_;
  first_ = hxcclSuccess;
  first_why_.clear();
  return r;
}

void HostWire::cancel_all() {
  for (int t : open_) ch_->cancel(t);
  open_.clear();
  first_ = hxcclSuccess;
  first_why_.clear();
}

hxcclResult_t HostWire::exchange(int to, const void* sbuf, size_t sbytes, int from, void* rbuf,
                                 size_t rbytes, bool fragment) {
  post_recv(from, rbuf, rbytes, kTagColl);
  if (hxcclResult_t r = post_send(to, sbuf, sbytes, kTagColl, fragment)) {
    cancel_all();
    return r;
  }
  return finish_all();
}

hxcclResult_t HostWire::send(int to, const void* buf, size_t bytes) {
  if (hxcclResult_t r = post_send(to, buf, bytes, kTagColl)) return r;
  return finish_all();
}

hxcclResult_t HostWire::recv(int from, void* buf, size_t bytes) {
  post_recv(from, buf, bytes, kTagColl);
  return finish_all();
}

}  // namespace hx
