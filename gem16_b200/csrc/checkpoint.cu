// Checkpoint loader of the quantized-contraction path: reads a safetensors container, validates an
// NVFP4 or FP8 module the way gem16's loader does (src/model/manifest.cpp:330-372: required tensors,
// exact dtypes and shapes; src/cuda/engine/target_model.cu:345-388: positive finite divisors) and binds
// it into the caller's device arena in this library's layouts -- the payload as stored, the block
// scales both compact (decode GEMV) and 128x4-interleaved (tcgen05 GEMMs).  A load-time component:
// it maps the file and uploads synchronously; nothing here is called on the launch path.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "common.cuh"

struct gemb_checkpoint {
  struct Tensor {
    std::string dtype;
    std::vector<uint64_t> shape;
    uint64_t begin = 0, end = 0;
  };
  std::map<std::string, Tensor> tensors;
  const uint8_t* map = nullptr;
  size_t map_bytes = 0;
  const uint8_t* data = nullptr;   // first byte behind the header
  size_t data_bytes = 0;
};

namespace gemb {
namespace {

// Just enough JSON for a safetensors header: objects, arrays, strings, non-negative integers.
struct Json {
  const char* p;
  const char* end;
  bool ok = true;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) {
    ws();
    if (p < end && *p == c) { ++p; return true; }
    return false;
  }
  std::string str() {
    std::string out;
    ws();
    if (p >= end || *p != '"') { ok = false; return out; }
    for (++p; p < end && *p != '"'; ++p) {
      if (*p == '\\' && p + 1 < end) ++p;
      out.push_back(*p);
    }
    if (p >= end) ok = false; else ++p;
    return out;
  }
  uint64_t num() {
    ws();
    if (p >= end || *p < '0' || *p > '9') { ok = false; return 0; }
    uint64_t v = 0;
    while (p < end && *p >= '0' && *p <= '9') v = v * 10 + static_cast<uint64_t>(*p++ - '0');
    return v;
  }
  void skip() {   // any value
    ws();
    if (p >= end) { ok = false; return; }
    if (*p == '"') { str(); return; }
    if (*p == '{' || *p == '[') {
      const char open = *p, close = open == '{' ? '}' : ']';
      ++p;
      if (eat(close)) return;
      do {
        if (open == '{') { str(); if (!eat(':')) { ok = false; return; } }
        skip();
      } while (ok && eat(','));
      if (!eat(close)) ok = false;
      return;
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;
  }
};

uint64_t dtype_bytes(const std::string& d) {
  if (d == "U8" || d == "I8" || d == "F8_E4M3" || d == "F8_E5M2" || d == "BOOL") return 1;
  if (d == "BF16" || d == "F16" || d == "I16" || d == "U16") return 2;
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  return 0;
}

uint64_t align256(uint64_t v) { return (v + 255) / 256 * 256; }

const gemb_checkpoint::Tensor* find(const gemb_checkpoint* c, const std::string& name) {
  auto it = c->tensors.find(name);
  return it == c->tensors.end() ? nullptr : &it->second;
}

struct Nvfp4Module {
  const gemb_checkpoint::Tensor *packed, *scale, *gw, *ga;
  uint64_t experts, rows, k;
};

int32_t check_nvfp4(const char* op, const gemb_checkpoint* c, const char* module, Nvfp4Module* m) {
  GEMB_REQUIRE(c != nullptr && module != nullptr, "%s: checkpoint and module name must be nonnull", op);
  const std::string base(module);
  m->packed = find(c, base + ".weight_packed");
  if (m->packed == nullptr) return fail(GEMB_NOT_FOUND, "%s: tensor %s.weight_packed is missing", op, module);
  m->scale = find(c, base + ".weight_scale");
  m->gw = find(c, base + ".weight_global_scale");
  m->ga = find(c, base + ".input_global_scale");
  if (!m->scale || !m->gw || !m->ga)
    return fail(GEMB_DATA_LOSS, "%s: NVFP4 tensor is missing a required scale tensor: %s", op, module);
  if (m->packed->dtype != "U8" || m->scale->dtype != "F8_E4M3" || m->gw->dtype != "F32" || m->ga->dtype != "F32")
    return fail(GEMB_DATA_LOSS, "%s: NVFP4 storage or scale dtype mismatch: %s", op, module);
  const size_t nd = m->packed->shape.size();
  if ((nd != 2 && nd != 3) || m->scale->shape.size() != nd)
    return fail(GEMB_DATA_LOSS, "%s: weight_packed / weight_scale must both be 2-D (or 3-D expert stacks): %s", op, module);
  m->experts = nd == 3 ? m->packed->shape[0] : 0;
  m->rows = m->packed->shape[nd - 2];
  m->k = m->packed->shape[nd - 1] * 2;
  if (m->k % 64 != 0 || m->rows % 8 != 0 || m->rows == 0 || m->k == 0)
    return fail(GEMB_DATA_LOSS, "%s: K must be a multiple of 64 and rows of 8: %s", op, module);
  if (m->scale->shape[nd - 2] != m->rows || m->scale->shape[nd - 1] * 16 != m->k || (nd == 3 && m->scale->shape[0] != m->experts))
    return fail(GEMB_DATA_LOSS, "%s: NVFP4 local scale shape does not describe groups of 16: %s", op, module);
  const std::vector<uint64_t> want{m->experts ? m->experts : 1};
  if (m->gw->shape != want || m->ga->shape != want)
    return fail(GEMB_DATA_LOSS, "%s: NVFP4 global scales must have shape [%llu]: %s", op,
                static_cast<unsigned long long>(want[0]), module);
  const float* gw = reinterpret_cast<const float*>(c->data + m->gw->begin);
  const float* ga = reinterpret_cast<const float*>(c->data + m->ga->begin);
  for (uint64_t i = 0; i < want[0]; ++i)
    if (!positive_finite(gw[i]) || !positive_finite(ga[i]))
      return fail(GEMB_DATA_LOSS, "%s: global divisors must be positive and finite: %s", op, module);
  const uint8_t* sc = c->data + m->scale->begin;
  for (uint64_t i = 0, n = m->scale->end - m->scale->begin; i < n; ++i)
    if ((sc[i] & 0x7F) == 0x7F) return fail(GEMB_DATA_LOSS, "%s: weight_scale holds an E4M3FN NaN encoding: %s", op, module);
  return GEMB_OK;
}

struct Nvfp4Plan {
  uint64_t packed, compact, interleaved, divisors, input_divisor, total;
};
Nvfp4Plan plan_nvfp4(const Nvfp4Module& m) {
  const uint64_t n = m.experts ? m.experts : 1;
  Nvfp4Plan p{};
  uint64_t cur = 0;
  p.packed = cur; cur += align256(n * m.rows * m.k / 2);
  p.compact = cur; cur += align256(n * m.rows * m.k / 16);
  p.interleaved = cur; cur += align256(n * gemb_interleaved_scale_bytes(m.rows, m.k));
  p.divisors = cur; cur += align256(n * 4);
  p.input_divisor = cur; cur += 256;
  p.total = cur;
  return p;
}

int32_t copy_up(const char* op, void* dst, const void* src, uint64_t bytes, cudaStream_t stream) {
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);   // the source is a pageable file mapping
  if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
  return GEMB_OK;
}

}  // namespace
}  // namespace gemb

using namespace gemb;

extern "C" {

int32_t gemb_checkpoint_open(const char* path, gemb_checkpoint** out) {
  const char* op = "gemb_checkpoint_open";
  GEMB_REQUIRE(path != nullptr && out != nullptr, "%s: path and result pointer must be nonnull", op);
  *out = nullptr;
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return fail(GEMB_IO_ERROR, "%s: cannot open %s", op, path);
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 8) {
    close(fd);
    return fail(GEMB_DATA_LOSS, "%s: %s is too short for a safetensors header", op, path);
  }
  void* map = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (map == MAP_FAILED) return fail(GEMB_IO_ERROR, "%s: cannot map %s", op, path);
  auto* c = new gemb_checkpoint;
  c->map = static_cast<const uint8_t*>(map);
  c->map_bytes = static_cast<size_t>(st.st_size);
  uint64_t header = 0;
  std::memcpy(&header, c->map, 8);
  auto bail = [&](int32_t code, const char* what) {
    gemb_checkpoint_close(c);
    return fail(code, "%s: %s: %s", op, path, what);
  };
  if (header > c->map_bytes - 8) return bail(GEMB_DATA_LOSS, "header length exceeds the file");
  c->data = c->map + 8 + header;
  c->data_bytes = c->map_bytes - 8 - header;
  Json j{reinterpret_cast<const char*>(c->map + 8), reinterpret_cast<const char*>(c->map + 8 + header)};
  if (!j.eat('{')) return bail(GEMB_DATA_LOSS, "header is not a JSON object");
  if (!j.eat('}')) {
    do {
      const std::string name = j.str();
      if (!j.ok || !j.eat(':')) return bail(GEMB_DATA_LOSS, "malformed header");
      if (name == "__metadata__") { j.skip(); continue; }
      gemb_checkpoint::Tensor t;
      if (!j.eat('{')) return bail(GEMB_DATA_LOSS, "malformed tensor entry");
      do {
        const std::string key = j.str();
        if (!j.eat(':')) return bail(GEMB_DATA_LOSS, "malformed tensor entry");
        if (key == "dtype") t.dtype = j.str();
        else if (key == "shape" || key == "data_offsets") {
          std::vector<uint64_t> v;
          if (!j.eat('[')) return bail(GEMB_DATA_LOSS, "malformed tensor entry");
          if (!j.eat(']')) {
            do v.push_back(j.num()); while (j.ok && j.eat(','));
            if (!j.eat(']')) return bail(GEMB_DATA_LOSS, "malformed tensor entry");
          }
          if (key == "shape") t.shape = v;
          else if (v.size() == 2) { t.begin = v[0]; t.end = v[1]; }
          else return bail(GEMB_DATA_LOSS, "data_offsets must hold two numbers");
        } else j.skip();
      } while (j.ok && j.eat(','));
      if (!j.ok || !j.eat('}')) return bail(GEMB_DATA_LOSS, "malformed tensor entry");
      const uint64_t size = dtype_bytes(t.dtype);
      if (size == 0) return bail(GEMB_UNSUPPORTED, "tensor with an unsupported dtype");
      uint64_t elements = 1;
      for (uint64_t d : t.shape) elements *= d;
      if (t.begin > t.end || t.end > c->data_bytes || t.end - t.begin != elements * size)
        return bail(GEMB_DATA_LOSS, "tensor with inconsistent shape / offsets");
      c->tensors.emplace(name, std::move(t));
    } while (j.ok && j.eat(','));
    if (!j.ok || !j.eat('}')) return bail(GEMB_DATA_LOSS, "malformed header");
  }
  *out = c;
  return GEMB_OK;
}

void gemb_checkpoint_close(gemb_checkpoint* checkpoint) {
  if (checkpoint == nullptr) return;
  if (checkpoint->map != nullptr) munmap(const_cast<uint8_t*>(checkpoint->map), checkpoint->map_bytes);
  delete checkpoint;
}

uint64_t gemb_checkpoint_nvfp4_bytes(const gemb_checkpoint* checkpoint, const char* module) {
  Nvfp4Module m;
  if (check_nvfp4("gemb_checkpoint_nvfp4_bytes", checkpoint, module, &m) != GEMB_OK) return 0;
  return plan_nvfp4(m).total;
}

int32_t gemb_checkpoint_bind_nvfp4(const gemb_checkpoint* checkpoint, const char* module, uint64_t rows,
                                   uint64_t contracting_elements, void* device_arena, uint64_t arena_bytes,
                                   gemb_nvfp4_binding* binding, gemb_stream_t stream) {
  const char* op = "gemb_checkpoint_bind_nvfp4";
  Nvfp4Module m;
  GEMB_TRY(check_nvfp4(op, checkpoint, module, &m));
  GEMB_REQUIRE(device_arena != nullptr && binding != nullptr && reinterpret_cast<uintptr_t>(device_arena) % 256 == 0,
               "%s: arena (256-byte aligned) and binding must be nonnull", op);
  if ((rows != 0 && rows != m.rows) || (contracting_elements != 0 && contracting_elements != m.k))
    return fail(GEMB_DATA_LOSS, "%s: unexpected NVFP4 tensor family: %s is [%llu, %llu]", op, module,
                static_cast<unsigned long long>(m.rows), static_cast<unsigned long long>(m.k));
  const Nvfp4Plan p = plan_nvfp4(m);
  GEMB_REQUIRE(arena_bytes >= p.total, "%s: arena too small (%llu bytes needed)", op, static_cast<unsigned long long>(p.total));
  GEMB_ENTER(op);
  uint8_t* base = static_cast<uint8_t*>(device_arena);
  const uint64_t n = m.experts ? m.experts : 1;
  GEMB_TRY(copy_up(op, base + p.packed, checkpoint->data + m.packed->begin, m.packed->end - m.packed->begin, stream));
  GEMB_TRY(copy_up(op, base + p.compact, checkpoint->data + m.scale->begin, m.scale->end - m.scale->begin, stream));
  GEMB_TRY(copy_up(op, base + p.divisors, checkpoint->data + m.gw->begin, n * 4, stream));
  GEMB_TRY(copy_up(op, base + p.input_divisor, checkpoint->data + m.ga->begin, 4, stream));
  const uint64_t per = gemb_interleaved_scale_bytes(m.rows, m.k);
  for (uint64_t e = 0; e < n; ++e)
    GEMB_TRY(gemb_nvfp4_interleave_scales(base + p.compact + e * m.rows * (m.k / 16), base + p.interleaved + e * per, m.rows,
                                          m.k, stream));
  const float* gw = reinterpret_cast<const float*>(checkpoint->data + m.gw->begin);
  const float* ga = reinterpret_cast<const float*>(checkpoint->data + m.ga->begin);
  *binding = gemb_nvfp4_binding{base + p.packed, base + p.compact, reinterpret_cast<const float*>(base + p.input_divisor),
                                ga[0], gw[0], m.rows, m.k, base + p.interleaved,
                                reinterpret_cast<const float*>(base + p.divisors), m.experts};
  return GEMB_OK;
}

uint64_t gemb_checkpoint_fp8_bytes(const gemb_checkpoint* checkpoint, const char* module) {
  if (checkpoint == nullptr || module == nullptr) return 0;
  const gemb_checkpoint::Tensor* w = find(checkpoint, std::string(module) + ".weight");
  if (w == nullptr || w->shape.size() != 2) return 0;
  return align256(w->shape[0] * w->shape[1]) + align256(w->shape[0] * 2);
}

int32_t gemb_checkpoint_bind_fp8(const gemb_checkpoint* checkpoint, const char* module, uint64_t rows,
                                 uint64_t contracting_elements, void* device_arena, uint64_t arena_bytes,
                                 gemb_fp8_binding* binding, gemb_stream_t stream) {
  const char* op = "gemb_checkpoint_bind_fp8";
  GEMB_REQUIRE(checkpoint != nullptr && module != nullptr && device_arena != nullptr && binding != nullptr &&
                   reinterpret_cast<uintptr_t>(device_arena) % 256 == 0,
               "%s: checkpoint, module, arena (256-byte aligned) and binding must be nonnull", op);
  const std::string base(module);
  const gemb_checkpoint::Tensor* w = find(checkpoint, base + ".weight");
  if (w == nullptr) return fail(GEMB_NOT_FOUND, "%s: tensor %s.weight is missing", op, module);
  const gemb_checkpoint::Tensor* s = find(checkpoint, base + ".weight_scale");
  if (s == nullptr) return fail(GEMB_DATA_LOSS, "%s: FP8 weight is missing its channel scale: %s", op, module);
  // src/model/manifest.cpp:366-372, src/cuda/engine/target_model.cu:345-358
  if (w->dtype != "F8_E4M3" || s->dtype != "BF16" || w->shape.size() != 2 ||
      s->shape != std::vector<uint64_t>{w->shape[0], 1} || (rows != 0 && rows != w->shape[0]) ||
      (contracting_elements != 0 && contracting_elements != w->shape[1]) || w->shape[1] % 16 != 0)
    return fail(GEMB_DATA_LOSS, "%s: FP8 weight/channel-scale schema mismatch: %s", op, module);
  const uint8_t* wb = checkpoint->data + w->begin;
  for (uint64_t i = 0, n = w->end - w->begin; i < n; ++i)
    if ((wb[i] & 0x7F) == 0x7F) return fail(GEMB_DATA_LOSS, "%s: weight holds an E4M3FN NaN encoding: %s", op, module);
  const uint64_t need = gemb_checkpoint_fp8_bytes(checkpoint, module);
  GEMB_REQUIRE(arena_bytes >= need, "%s: arena too small (%llu bytes needed)", op, static_cast<unsigned long long>(need));
  GEMB_ENTER(op);
  uint8_t* d = static_cast<uint8_t*>(device_arena);
  uint8_t* d_scales = d + align256(w->shape[0] * w->shape[1]);
  GEMB_TRY(copy_up(op, d, wb, w->end - w->begin, stream));
  GEMB_TRY(copy_up(op, d_scales, checkpoint->data + s->begin, s->end - s->begin, stream));
  *binding = gemb_fp8_binding{d, reinterpret_cast<const uint16_t*>(d_scales), w->shape[0], w->shape[1]};
  return GEMB_OK;
}

}  // extern "C"
