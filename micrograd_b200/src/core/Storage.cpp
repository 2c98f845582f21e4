// detail::Storage — device buffer + lazily materialised host mirror.
#include "micrograd/detail/Storage.h"

#include <stdexcept>
#include <string>

#include "mg_cuda.h"

namespace micrograd::detail {

namespace {
constexpr size_t kKeepHostElems = 4096;
unsigned long long g_device_epoch = 0;
}

unsigned long long device_epoch() { return g_device_epoch; }
void advance_device_epoch() { g_device_epoch++; }

void check(int rc, const char *what) {
  if (rc != MG_OK) {
    throw std::runtime_error(std::string(what) + ": " + mg_last_error());
  }
}

Storage::~Storage() {
  if (mg_device() < 0) {
    // The device context is gone (mg_shutdown, or static destruction order at
    // exit): its pool and events went with it, and touching the ABI here would
    // bring a whole new context up only to fail the lookups.
    return;
  }
  if (pending_upload_ >= 0) {
    // never read: still order the free after the copy
    mg_compute_wait_event(pending_upload_);
    mg_event_destroy(pending_upload_);
  }
  if (dev_ && owns_dev_) {
    mg_free(dev_);
  }
}

void Storage::init_zero(size_t n) {
  size_ = n;
  zero_ = true;
  dev_valid_ = false;
  host_valid_ = false;
}

void Storage::ensure_device_buffer() {
  if (!dev_) {
    check(mg_alloc(size_, &dev_), "device allocation");
    owns_dev_ = true;
  }
}

void Storage::init_from_host(std::vector<double> &&values) {
  size_ = values.size();
  ensure_device_buffer();
  // A copy from pageable memory has been staged when the call returns, so the
  // temporary can be released right away; the device copy is the only one kept.
  check(mg_upload(dev_, values.data(), size_), "upload");
  zero_ = false;
  dev_valid_ = true;
  // Small tensors (labels, scalars, single samples) keep their host copy, so
  // reading them back through at()/data() needs no device round trip.
  if (size_ <= kKeepHostElems) {
    host_ = std::move(values);
    host_valid_ = true;
    host_epoch_ = g_device_epoch;
  } else {
    host_valid_ = false;
  }
}

void Storage::settle_upload() {
  if (pending_upload_ >= 0) {
    check(mg_compute_wait_event(pending_upload_), "wait for upload");
    check(mg_event_destroy(pending_upload_), "event destroy");
    pending_upload_ = -1;
  }
}

void Storage::init_from_pointer(const double *values, size_t n) {
  size_ = n;
  ensure_device_buffer();
  check(mg_upload_async(dev_, values, n, &pending_upload_), "upload");
  zero_ = false;
  dev_valid_ = true;
  host_valid_ = false;
}

void Storage::sync_device_from_host() {
  ensure_device_buffer();
  check(mg_upload(dev_, host_.data(), size_), "upload");
  dev_valid_ = true;
}

void Storage::settle_exchange() {
  if (comm_pending_) {
    // An all-reduce on the communication stream is still writing this buffer (peers
    // store into it too): reads on the compute stream wait for it on the device.
    check(mg_comm_join(), "comm join");
    comm_pending_ = false;
  }
}

void Storage::sync_host_from_device() {
  settle_exchange();
  host_.resize(size_);
  double mirrored = 0.0;
  if (fetch_mirror(&mirrored)) {
    host_[0] = mirrored;
  } else {
    check(mg_download(host_.data(), dev_, size_), "download");
  }
  host_valid_ = true;
  host_epoch_ = g_device_epoch;
}

// A one-element result is copied to pinned host memory right behind its producer,
// so that a host read some kernels later waits for that copy and not for the
// whole queue (a training loop reads its loss after enqueueing the backward pass).
void Storage::mirror_async() {
  if (size_ != 1 || zero_ || !dev_valid_ || !dev_) {
    return;
  }
  check(mg_scalar_mirror(dev_, &mirror_ticket_), "scalar mirror");
  mirror_stamp_ = write_stamp_;
}

bool Storage::fetch_mirror(double *value) {
  if (mirror_ticket_ == 0 || mirror_stamp_ != write_stamp_ || size_ != 1) {
    return false;  // no mirror, or the contents were rewritten since
  }
  int expired = 0;
  check(mg_scalar_fetch(mirror_ticket_, value, &expired), "scalar fetch");
  return expired == 0;
}

const double *Storage::device_read() {
  settle_upload();
  if (zero_) {
    ensure_device_buffer();
    check(mg_fill(dev_, 0.0, size_), "fill");
    zero_ = false;
    dev_valid_ = true;
    host_valid_ = false;
  } else if (!dev_valid_) {
    sync_device_from_host();
  }
  return dev_;
}

double *Storage::device_overwrite() {
  write_stamp_++;
  settle_upload();
  ensure_device_buffer();
  zero_ = false;
  dev_valid_ = true;
  host_valid_ = false;
  return dev_;
}

double *Storage::device_accumulate(bool *store) {
  write_stamp_++;
  settle_upload();
  if (zero_) {
    ensure_device_buffer();
    *store = true;
    zero_ = false;
    dev_valid_ = true;
    host_valid_ = false;
    return dev_;
  }
  *store = false;
  if (!dev_valid_) {
    sync_device_from_host();
  }
  host_valid_ = false;
  return dev_;
}

double *Storage::device_update() {
  write_stamp_++;
  device_read();
  host_valid_ = false;
  return dev_;
}

void Storage::set_zero() {
  write_stamp_++;
  settle_upload();
  zero_ = true;
  dev_valid_ = false;
  host_valid_ = false;
}

void Storage::fill(double value) {
  write_stamp_++;
  settle_upload();
  ensure_device_buffer();
  check(mg_fill(dev_, value, size_), "fill");
  zero_ = false;
  dev_valid_ = true;
  host_valid_ = false;
}

std::vector<double> &Storage::host_mutable() {
  host_const();  // (before the stamp moves: a pending scalar mirror is still current here)
  if (zero_) {
    zero_ = false;  // the zeros just written to host_ are now the contents
    host_valid_ = true;
  }
  write_stamp_++;
  // The caller may write through the reference at any later time, so the host
  // vector is the authority until a kernel needs the values again.
  dev_valid_ = false;
  return host_;
}

const std::vector<double> &Storage::host_const() {
  settle_upload();
  if (zero_) {
    // A read does not end the logical-zero state: the next accumulation is still
    // a plain store and no buffer has to be filled.
    host_.assign(size_, 0.0);
  } else if (!host_valid_ || (dev_valid_ && host_epoch_ != g_device_epoch)) {
    // (second case: a recorded step was replayed since the host copy was taken)
    sync_host_from_device();
  }
  return host_;
}

double Storage::peek(size_t index) {
  settle_upload();
  if (zero_ || index >= size_) {
    return 0.0;
  }
  if (host_valid_ && !(dev_valid_ && host_epoch_ != g_device_epoch)) {
    return host_[index];
  }
  double v = 0.0;
  if (fetch_mirror(&v)) {
    return v;
  }
  settle_exchange();
  check(mg_download(&v, dev_ + index, 1), "download");
  return v;
}

void Storage::upload_in_place(const double *values) {
  write_stamp_++;
  settle_upload();
  ensure_device_buffer();
  check(mg_upload(dev_, values, size_), "upload");
  zero_ = false;
  dev_valid_ = true;
  host_valid_ = false;
}

void Storage::prefetch_in_place(const double *values) {
  write_stamp_++;
  settle_upload();  // an earlier prefetch into the same buffer is ordered first
  ensure_device_buffer();
  // The copy stream waits for everything enqueued on the compute stream so far
  // (every earlier reader of this buffer), copies, and the next kernel that
  // touches the buffer waits for the copy (settle_upload).
  check(mg_upload_async(dev_, values, size_, &pending_upload_), "upload");
  zero_ = false;
  dev_valid_ = true;
  host_valid_ = false;
}

void Storage::rehome(double *slice, std::shared_ptr<void> keepalive) {
  settle_upload();
  if (!zero_) {
    if (dev_valid_) {
      check(mg_copy(slice, dev_, size_), "copy");
    } else {
      check(mg_upload(slice, host_.data(), size_), "upload");
      dev_valid_ = true;
    }
  }
  if (dev_ && owns_dev_) {
    check(mg_free(dev_), "free");
  }
  dev_ = slice;
  owns_dev_ = false;
  keepalive_ = std::move(keepalive);
}

void Storage::adopt(double *slice, std::shared_ptr<void> keepalive) {
  settle_upload();
  if (dev_ && owns_dev_) {
    check(mg_free(dev_), "free");
  }
  dev_ = slice;
  owns_dev_ = false;
  keepalive_ = std::move(keepalive);
  zero_ = false;
  dev_valid_ = true;
  host_valid_ = false;
  write_stamp_++;
}

DeviceInts::DeviceInts(const int *host_values, size_t n) : n_(n) {
  check(mg_alloc_i32(n, &dev_), "device allocation");
  check(mg_upload_i32(dev_, host_values, n), "upload");
}

DeviceInts::DeviceInts(size_t n) : n_(n) { check(mg_alloc_i32(n, &dev_), "device allocation"); }

DeviceInts::~DeviceInts() {
  if (dev_) {
    mg_free_i32(dev_);
  }
}

}  // namespace micrograd::detail
