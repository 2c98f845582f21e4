// IDX file reader (reference: src/mnist.cpp).  Same file handling as the
// reference — 16-byte image header and 8-byte label header are skipped, one
// byte per pixel scaled by 1/255, one byte per label — but the files are read
// with two block reads, the pixel bytes are uploaded as bytes and divided by
// 255.0 on the device (one IEEE division per pixel, the same value the host
// computes), and the labels follow in a second upload.
#include "micrograd/mnist.h"

#include <fstream>
#include <stdexcept>

#include "internal.h"
#include "mg_cuda.h"

using micrograd::detail::check;

namespace {

struct RawMnist {
  std::vector<unsigned char> pixels;  // [count][784], raw bytes
  std::vector<unsigned char> labels;
};

RawMnist read_idx(const std::string &images_path, const std::string &labels_path, int sample_count) {
  RawMnist raw;
  const size_t count = sample_count > 0 ? static_cast<size_t>(sample_count) : 0;
  std::ifstream images(images_path, std::ios::binary);
  std::ifstream labels(labels_path, std::ios::binary);
  std::vector<unsigned char> &bytes = raw.pixels;
  bytes.assign(count * 784, 0);
  raw.labels.assign(count, 0);
  // Like the reference, a missing or short file is not an error: unread samples
  // keep zero pixels and label 0.
  if (images.is_open()) {
    images.seekg(16);
    images.read(reinterpret_cast<char *>(bytes.data()), static_cast<std::streamsize>(bytes.size()));
  }
  if (labels.is_open()) {
    labels.seekg(8);
    labels.read(reinterpret_cast<char *>(raw.labels.data()),
                static_cast<std::streamsize>(raw.labels.size()));
  }
  return raw;
}

struct DeviceBlock {
  double *ptr = nullptr;
  ~DeviceBlock() { mg_free(ptr); }
};

}  // namespace

MNISTData load_mnist(const std::string &images_path, const std::string &labels_path,
                     int sample_count) {
  RawMnist raw = read_idx(images_path, labels_path, sample_count);
  const size_t count = raw.labels.size();
  MNISTData data;
  if (count == 0) {
    return data;
  }
  std::vector<double> one_hot(count * 10, 0.0);
  for (size_t i = 0; i < count; i++) {
    one_hot[i * 10 + (raw.labels[i] % 10)] = 1.0;
  }
  auto image_block = std::make_shared<DeviceBlock>();
  auto label_block = std::make_shared<DeviceBlock>();
  check(mg_alloc(count * 784, &image_block->ptr), "device allocation");
  check(mg_alloc(count * 10, &label_block->ptr), "device allocation");
  check(mg_upload_u8_scaled(image_block->ptr, raw.pixels.data(), count * 784, 255.0), "upload");
  check(mg_upload(label_block->ptr, one_hot.data(), count * 10), "upload");
  data.images.reserve(count);
  data.labels.reserve(count);
  for (size_t i = 0; i < count; i++) {
    auto image = std::make_shared<Tensor>(std::vector<size_t>{1, 784});
    auto label = std::make_shared<Tensor>(std::vector<size_t>{1, 10});
    micrograd::detail::TensorAccess::data(*image).adopt(image_block->ptr + i * 784, image_block);
    micrograd::detail::TensorAccess::data(*label).adopt(label_block->ptr + i * 10, label_block);
    data.images.push_back(std::move(image));
    data.labels.push_back(std::move(label));
  }
  return data;
}

MNISTBatch load_mnist_batched(const std::string &images_path, const std::string &labels_path,
                              int sample_count) {
  RawMnist raw = read_idx(images_path, labels_path, sample_count);
  const size_t count = raw.labels.size();
  std::vector<double> ids(count);
  for (size_t i = 0; i < count; i++) {
    ids[i] = static_cast<double>(raw.labels[i]);
  }
  MNISTBatch batch;
  batch.images = std::make_shared<Tensor>(std::vector<size_t>{count, 784});
  if (count > 0) {
    check(mg_upload_u8_scaled(micrograd::detail::TensorAccess::data(*batch.images).device_overwrite(),
                              raw.pixels.data(), count * 784, 255.0),
          "upload");
  }
  batch.labels = std::make_shared<Tensor>(std::vector<size_t>{count}, std::move(ids));
  return batch;
}
