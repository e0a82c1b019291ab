// Parameter checkpoints of the fused nets.  The reference keeps its parameters only in the device
// buffers of its four static Layer objects (main.cu:17-20, filled at layer.cu:19-27) and loses them
// when the process exits; this file writes and reads the arena as a small self-describing file.
//
// Layout (little-endian, as every machine this library runs on):
//   bytes 0..7    magic "CNNB200P"
//   u32           version (1)
//   u32           kind: 0 = the reference's 28x28 net, 1 = widened net
//   u32 H, u32 F  input side and number of feature maps
//   u32           parameter count
//   u32           seed the net was created with (0 for widened nets)
//   f32[count]    the arena, in the order the header of the C ABI documents
//   u64           FNV-1a of every byte before it
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "wide.cuh"

namespace cnn {
namespace {

constexpr char kMagic[8] = {'C', 'N', 'N', 'B', '2', '0', '0', 'P'};
constexpr uint32_t kVersion = 1;

struct Header {
  char magic[8];
  uint32_t version, kind, H, F, count, seed;
};
static_assert(sizeof(Header) == 32, "checkpoint header is 32 bytes");

uint64_t fnv1a(const unsigned char* p, size_t n, uint64_t h = 1469598103934665603ull) {
  for (size_t i = 0; i < n; ++i) {
    h ^= p[i];
    h *= 1099511628211ull;
  }
  return h;
}

int save_arena(const char* path, uint32_t kind, uint32_t H, uint32_t F, uint32_t seed, const float* d_params,
               uint32_t count) {
  std::vector<unsigned char> buf(sizeof(Header) + sizeof(float) * (size_t)count + sizeof(uint64_t));
  Header h;
  std::memcpy(h.magic, kMagic, 8);
  h.version = kVersion; h.kind = kind; h.H = H; h.F = F; h.count = count; h.seed = seed;
  std::memcpy(buf.data(), &h, sizeof(h));
  CNN_CUDA(cudaDeviceSynchronize());   // updates in flight on any stream are part of what is saved
  CNN_CUDA(cudaMemcpy(buf.data() + sizeof(h), d_params, sizeof(float) * (size_t)count, cudaMemcpyDeviceToHost));
  const uint64_t sum = fnv1a(buf.data(), buf.size() - sizeof(uint64_t));
  std::memcpy(buf.data() + buf.size() - sizeof(uint64_t), &sum, sizeof(sum));
  FILE* f = std::fopen(path, "wb");
  if (!f) {
    set_error("checkpoint: cannot open '%s' for writing", path);
    return CNN_ERR_INVALID;
  }
  const size_t wrote = std::fwrite(buf.data(), 1, buf.size(), f);
  const int closed = std::fclose(f);
  if (wrote != buf.size() || closed != 0) {
    set_error("checkpoint: short write to '%s'", path);
    return CNN_ERR_INVALID;
  }
  return CNN_OK;
}

int load_arena(const char* path, uint32_t kind, uint32_t H, uint32_t F, float* d_params, uint32_t count,
               uint32_t* seed_out) {
  FILE* f = std::fopen(path, "rb");
  if (!f) {
    set_error("checkpoint: cannot open '%s'", path);
    return CNN_ERR_INVALID;
  }
  std::vector<unsigned char> buf(sizeof(Header) + sizeof(float) * (size_t)count + sizeof(uint64_t) + 1);
  const size_t got = std::fread(buf.data(), 1, buf.size(), f);
  std::fclose(f);
  Header h;
  if (got < sizeof(Header)) {
    set_error("checkpoint: '%s' is shorter than a header", path);
    return CNN_ERR_INVALID;
  }
  std::memcpy(&h, buf.data(), sizeof(h));
  if (std::memcmp(h.magic, kMagic, 8) != 0) {
    set_error("checkpoint: '%s' does not start with the magic CNNB200P", path);
    return CNN_ERR_INVALID;
  }
  if (h.version != kVersion) {
    set_error("checkpoint: '%s' has version %u, this library reads version %u", path, h.version, kVersion);
    return CNN_ERR_INVALID;
  }
  if (h.kind != kind || h.H != H || h.F != F || h.count != count) {
    set_error("checkpoint: '%s' holds kind %u, H %u, F %u, %u parameters; the net is kind %u, H %u, F %u, %u", path,
              h.kind, h.H, h.F, h.count, kind, H, F, count);
    return CNN_ERR_INVALID;
  }
  const size_t want = sizeof(Header) + sizeof(float) * (size_t)count + sizeof(uint64_t);
  if (got != want) {
    set_error("checkpoint: '%s' has %zu bytes, expected %zu", path, got, want);
    return CNN_ERR_INVALID;
  }
  uint64_t stored;
  std::memcpy(&stored, buf.data() + want - sizeof(uint64_t), sizeof(stored));
  if (stored != fnv1a(buf.data(), want - sizeof(uint64_t))) {
    set_error("checkpoint: checksum mismatch in '%s'", path);
    return CNN_ERR_INVALID;
  }
  // same ordering as cnn_net_set_params: nothing in flight sees a mixture, and the upload has landed
  // before a launch on a non-blocking stream
  CNN_CUDA(cudaDeviceSynchronize());
  CNN_CUDA(cudaMemcpy(d_params, buf.data() + sizeof(Header), sizeof(float) * (size_t)count, cudaMemcpyHostToDevice));
  CNN_CUDA(cudaDeviceSynchronize());
  if (seed_out) *seed_out = h.seed;
  return CNN_OK;
}

}  // namespace
}  // namespace cnn

using namespace cnn;

extern "C" {

int cnn_net_save(cnn_net* net, const char* path) {
  CNN_REQUIRE(net && path, "cnn_net_save: NULL argument");
  return save_arena(path, 0, kH, kF, net->seed, net->d_params, kNParams);
}

int cnn_net_load(cnn_net* net, const char* path) {
  CNN_REQUIRE(net && path, "cnn_net_load: NULL argument");
  return load_arena(path, 0, kH, kF, net->d_params, kNParams, &net->seed);
}

int cnn_wide_save(cnn_wide* w, const char* path) {
  CNN_REQUIRE(w && path, "cnn_wide_save: NULL argument");
  return save_arena(path, 1, (uint32_t)w->d.H, (uint32_t)w->d.F, 0, w->d_params, (uint32_t)w->d.n_params);
}

int cnn_wide_load(cnn_wide* w, const char* path) {
  CNN_REQUIRE(w && path, "cnn_wide_load: NULL argument");
  return load_arena(path, 1, (uint32_t)w->d.H, (uint32_t)w->d.F, w->d_params, (uint32_t)w->d.n_params, nullptr);
}

}  // extern "C"
