#pragma once
// Device-resident fp64 buffer with a lazily materialised host mirror.
//
// Stands in for the reference's `std::vector<double> data_, grad_`
// (include/micrograd/Tensor.h:55-56).  The authoritative copy is in GPU memory;
// a host std::vector appears only when the public accessors data()/grad()/at()
// ask for one.  Those accessors hand out mutable references, so once the host
// view has been lent the device copy is treated as stale and is refreshed from
// the host vector before the next kernel touches it.

#include <cstddef>
#include <memory>
#include <vector>

namespace micrograd::detail {

class Storage {
public:
  Storage() = default;
  ~Storage();
  Storage(const Storage &) = delete;
  Storage &operator=(const Storage &) = delete;

  // Logical all-zero contents of `n` elements; nothing is allocated yet.
  void init_zero(size_t n);
  // Takes ownership of host values and uploads them.
  void init_from_host(std::vector<double> &&values);
  // Uploads `n` values straight from caller memory (may be pinned) on the copy
  // stream, so the transfer overlaps kernels already enqueued; the first kernel
  // that touches the buffer waits for it on the device.  The caller keeps
  // `values` unchanged until then.
  void init_from_pointer(const double *values, size_t n);

  size_t size() const { return size_; }
  bool is_zero() const { return zero_; }

  // Device pointer whose contents are current; for kernels that only read.
  const double *device_read();
  // Device pointer the caller will overwrite completely.
  double *device_overwrite();
  // Device pointer for `+=`.  If the contents are logically zero, *store is set
  // and the caller must write every element instead of accumulating.
  double *device_accumulate(bool *store);
  // Device pointer for in-place update of current contents.
  double *device_update();

  void set_zero();          // back to logical zeros (keeps any buffer)
  void fill(double value);  // every element := value, on the device

  // Host views.  The mutable one marks the device copy stale.
  std::vector<double> &host_mutable();
  const std::vector<double> &host_const();
  double peek(size_t index);  // one element, without lending the host view
  // For a one-element buffer whose producer has just been enqueued: start an
  // asynchronous copy to the host, so a later read need not wait for kernels
  // enqueued after the producer.  No effect on larger buffers.
  void mirror_async();

  // Overwrites the contents with `size()` values from caller memory, in the device
  // buffer this storage already has (its address does not change, which a recorded
  // step relies on).
  void upload_in_place(const double *values);
  void prefetch_in_place(const double *values);  // the same through the copy stream

  // Moves the contents into caller-owned device memory (a slice of a flat
  // parameter/gradient buffer) and uses that memory from now on.
  // `keepalive` owns that memory.
  void rehome(double *slice, std::shared_ptr<void> keepalive);
  // Uses caller-owned device memory that already holds the values (a slice of a
  // larger upload); `keepalive` owns that memory.
  void adopt(double *slice, std::shared_ptr<void> keepalive);
  // True when the device buffer holds the current values (not logical zeros,
  // not superseded by a lent host view).
  bool device_current() const { return !zero_ && dev_valid_; }
  // Counts every hand-out of the contents for writing (device or host); lets a
  // caller detect that nobody has touched the buffer since it last looked.
  unsigned long long write_stamp() const { return write_stamp_; }
  // Marks the buffer as the target of an all-reduce still running on the
  // communication stream; the next host read joins that stream first.
  void set_exchange_pending(bool pending) { comm_pending_ = pending; }

private:
  void ensure_device_buffer();
  void settle_upload();  // make the compute stream wait for a pending prefetch
  void settle_exchange();  // make the compute stream wait for a pending all-reduce
  void sync_device_from_host();
  void sync_host_from_device();
  bool fetch_mirror(double *value);  // true: *value is the mirrored, still current element

  size_t size_ = 0;
  double *dev_ = nullptr;
  bool owns_dev_ = true;
  std::shared_ptr<void> keepalive_;
  bool zero_ = true;         // logically all zeros; dev_/host_ contents irrelevant
  bool dev_valid_ = false;   // dev_ holds the current values
  bool host_valid_ = false;  // host_ holds the current values
  unsigned long long write_stamp_ = 0;
  unsigned long long host_epoch_ = 0;  // device epoch at which host_ was last made current
  bool comm_pending_ = false;  // an all-reduce on the communication stream targets dev_
  int pending_upload_ = -1;  // event id of a prefetch the compute stream has not waited for
  unsigned long long mirror_ticket_ = 0;  // pending scalar mirror (0: none)
  unsigned long long mirror_stamp_ = 0;   // write_stamp_ when the mirror was started
  std::vector<double> host_;
};

// Device-side int buffer (class ids), shared by graph closures.
class DeviceInts {
public:
  DeviceInts(const int *host_values, size_t n);
  explicit DeviceInts(size_t n);
  ~DeviceInts();
  DeviceInts(const DeviceInts &) = delete;
  DeviceInts &operator=(const DeviceInts &) = delete;
  int *get() const { return dev_; }
  size_t size() const { return n_; }

private:
  int *dev_ = nullptr;
  size_t n_ = 0;
};

// Counts replays of recorded steps.  A replay rewrites device buffers without
// passing through the host-side bookkeeping, so a host copy taken in an earlier
// epoch is stale whenever the device buffer is the authority.
unsigned long long device_epoch();
void advance_device_epoch();

// Throws std::runtime_error carrying mg_last_error() when rc != 0.
void check(int rc, const char *what);

}  // namespace micrograd::detail
