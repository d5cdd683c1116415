// Readers of the reference's on-disk data and parameter formats, feeding the host programs.
//
//   float data set   <name>_{train,test}.bin = raw float32 samples back to back, <name>_{train,test}_target.bin = one raw
//                    int32 label per sample; samples are used as (x - mean) / std
//                    (DataLoader, src/main/scala/lantern/TensorDataLoader.scala:64-108; Tensor.normalize,
//                    src/main/scala/lantern/TensorDifferentiation.scala:936-945).
//   CIFAR binary     records of 1 label byte + sample_bytes pixel bytes (3072 for CIFAR-10); x = byte / 255
//                    (Cifar10DataLoader, TensorDataLoader.scala:110-139).
//   parameter file   <model>.onnx.bin = the model's float32 tensors back to back, unpadded, in declaration order;
//                    a tensor is addressed by its offset in floats (ParameterWriter / ParameterReader,
//                    src/main/scala/lantern/ONNXLib.scala:157-185).
// The reference decodes a whole file into a float array up front and hands out slices of it; here the file stays
// mapped as it is on disk and one batch at a time is decoded straight into the pinned staging buffer of the step
// that will upload it, while the device runs the step before (Model::submit in models.cpp).
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

namespace lantern_host {

struct MappedFile {
  const uint8_t* data = nullptr; size_t bytes = 0; int fd = -1;
  bool open(const char* path) {
    fd = ::open(path, O_RDONLY);
    if (fd < 0) return false;
    struct stat st;
    if (fstat(fd, &st) != 0) { close(); return false; }
    bytes = (size_t)st.st_size;
    if (bytes) {
      void* p = mmap(nullptr, bytes, PROT_READ, MAP_PRIVATE, fd, 0);
      if (p == MAP_FAILED) { close(); return false; }
      data = (const uint8_t*)p;
    }
    return true;
  }
  void close() {
    if (data) munmap((void*)data, bytes);
    if (fd >= 0) ::close(fd);
    data = nullptr; bytes = 0; fd = -1;
  }
};

struct Loader {
  enum Kind { FLOATS = 0, CIFAR = 1 };
  Kind kind = FLOATS;
  MappedFile samples, targets;
  int64_t sample_count = 0;     // floats (FLOATS) or pixel bytes (CIFAR) per sample
  int64_t length = 0;           // samples in the file
  float mean = 0.f, stdev = 1.f;
  std::string error;

  bool open_floats(const char* data_path, const char* target_path, int64_t floats_per_sample, float m, float s) {
    kind = FLOATS; sample_count = floats_per_sample; mean = m; stdev = s;
    if (floats_per_sample <= 0) { error = "sample size must be positive"; return false; }
    if (!samples.open(data_path)) { error = std::string("cannot map ") + data_path; return false; }
    if (!targets.open(target_path)) { error = std::string("cannot map ") + target_path; return false; }
    length = (int64_t)(targets.bytes / 4);
    // the reference asserts the same after walking the file: "Data length doesn't match" (TensorDataLoader.scala:95)
    if ((int64_t)(samples.bytes / 4) != length * floats_per_sample) { error = "data length does not match the number of targets"; return false; }
    return true;
  }
  bool open_cifar(const char* path, int64_t bytes_per_sample) {
    kind = CIFAR; sample_count = bytes_per_sample;
    if (bytes_per_sample <= 0) { error = "sample size must be positive"; return false; }
    if (!samples.open(path)) { error = std::string("cannot map ") + path; return false; }
    length = (int64_t)(samples.bytes / (size_t)(bytes_per_sample + 1));      // a trailing partial record is ignored, as in the reference
    return true;
  }
  int64_t batches(int batch) const { return batch > 0 ? length / batch : 0; }  // the last partial batch is dropped (foreachBatch)
  // Decode batch `index` (samples index*batch .. +batch) into x (batch * sample_count floats) and y (batch labels).
  bool fill(int64_t index, int batch, float* x, int32_t* y) const {
    if (index < 0 || index >= batches(batch)) return false;
    const int64_t first = index * batch;
    if (kind == FLOATS) {
      const float* src = (const float*)samples.data + first * sample_count;
      const int64_t n = (int64_t)batch * sample_count;
      if (mean == 0.f && stdev == 1.f) memcpy(x, src, (size_t)n * 4);
      else for (int64_t i = 0; i < n; ++i) x[i] = (src[i] - mean) / stdev;
      memcpy(y, (const int32_t*)targets.data + first, (size_t)batch * 4);
    } else {
      const uint8_t* rec = samples.data + first * (sample_count + 1);
      for (int b = 0; b < batch; ++b, rec += sample_count + 1) {
        y[b] = (int32_t)rec[0];
        float* dst = x + (int64_t)b * sample_count;
        for (int64_t j = 0; j < sample_count; ++j) dst[j] = (float)rec[1 + j] / 255.0f;
      }
    }
    return true;
  }
  void close() { samples.close(); targets.close(); }
};

}  // namespace lantern_host
