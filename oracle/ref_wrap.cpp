// C entry points around the UNMODIFIED gem16 CPU numeric sources (src/numeric/nvfp4.cpp,
// src/numeric/fp8.cpp, src/numeric/layer.cpp), which the build recipe compiles from the reference tree where it lies.
// TEST INFRASTRUCTURE ONLY: used to pin gemb_oracle.cpp and as the timed CPU reference arm.
// The reference functions are called as they are; this file only loops over rows with threads.
#include <atomic>
#include <cstdint>
#include <span>
#include <thread>
#include <vector>

#include "gem16/fp8.h"
#include "gem16/layer.h"
#include "gem16/nvfp4.h"

namespace {
template <typename F>
void parallel_for(uint64_t n, int threads, F fn) {
  if (threads <= 1 || n < 2) {
    for (uint64_t i = 0; i < n; ++i) fn(i);
    return;
  }
  std::atomic<uint64_t> next{0};
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([&] {
      for (;;) {
        uint64_t i = next.fetch_add(1);
        if (i >= n) break;
        fn(i);
      }
    });
  for (auto& th : pool) th.join();
}
}  // namespace

extern "C" {

float ref_e2m1_decode(uint8_t nib) { return gem16::nvfp4::DecodeE2M1(nib); }
int ref_e2m1_encode(float v) {
  auto r = gem16::nvfp4::EncodeE2M1(v);
  return r.ok() ? r.value() : -1;
}
float ref_e4m3_decode(uint8_t b) { return gem16::nvfp4::DecodeE4M3Fn(b); }
int ref_e4m3_encode(float v) {
  auto r = gem16::nvfp4::EncodeE4M3Fn(v);
  return r.ok() ? r.value() : -1;
}
float ref_bf16_decode(uint16_t b) { return gem16::fp8::DecodeBf16(b); }

// gem16::nvfp4::QuantizeActivation per token.  Returns the reference StatusCode of the first
// failing token (0 = ok).
int ref_nvfp4_quantize(const float* x, uint64_t tokens, uint64_t k, float g, uint8_t* packed,
                       uint8_t* scales, int threads) {
  std::atomic<int> status{0};
  parallel_for(tokens, threads, [&](uint64_t t) {
    auto q = gem16::nvfp4::QuantizeActivation(std::span<const float>(x + t * k, k), g);
    if (!q.ok()) {
      status = static_cast<int>(q.status().code());
      return;
    }
    std::copy(q.value().packed_e2m1.begin(), q.value().packed_e2m1.end(), packed + t * (k / 2));
    std::copy(q.value().block_scales_e4m3fn.begin(), q.value().block_scales_e4m3fn.end(),
              scales + t * (k / 16));
  });
  return status.load();
}

// gem16::nvfp4::ReferenceDotProduct for every (token, row).
int ref_nvfp4_matmul(const uint8_t* a_packed, const uint8_t* a_scales, const uint8_t* w_packed,
                     const uint8_t* w_scales, uint64_t tokens, uint64_t rows, uint64_t k, float ga,
                     float gw, double* out, int threads) {
  std::vector<gem16::nvfp4::QuantizedActivation> acts(tokens);
  for (uint64_t t = 0; t < tokens; ++t) {
    acts[t].logical_elements = k;
    acts[t].global_divisor = ga;
    acts[t].packed_e2m1.assign(a_packed + t * (k / 2), a_packed + (t + 1) * (k / 2));
    acts[t].block_scales_e4m3fn.assign(a_scales + t * (k / 16), a_scales + (t + 1) * (k / 16));
  }
  std::atomic<int> status{0};
  parallel_for(rows, threads, [&](uint64_t r) {
    std::span<const uint8_t> wp(w_packed + r * (k / 2), k / 2);
    std::span<const uint8_t> ws(w_scales + r * (k / 16), k / 16);
    for (uint64_t t = 0; t < tokens; ++t) {
      auto d = gem16::nvfp4::ReferenceDotProduct(acts[t], wp, ws, gw);
      if (!d.ok()) {
        status = static_cast<int>(d.status().code());
        return;
      }
      out[t * rows + r] = d.value();
    }
  });
  return status.load();
}

int ref_fp8_quantize(const float* x, uint64_t tokens, uint64_t k, uint8_t* q, float* scales,
                     int threads) {
  std::atomic<int> status{0};
  parallel_for(tokens, threads, [&](uint64_t t) {
    auto r = gem16::fp8::QuantizeToken(std::span<const float>(x + t * k, k));
    if (!r.ok()) {
      status = static_cast<int>(r.status().code());
      return;
    }
    std::copy(r.value().values_e4m3fn.begin(), r.value().values_e4m3fn.end(), q + t * k);
    scales[t] = r.value().scale;
  });
  return status.load();
}

int ref_fp8_matmul(const uint8_t* a, const float* a_scales, const uint8_t* w,
                   const uint16_t* w_scales_bf16, uint64_t tokens, uint64_t rows, uint64_t k,
                   double* out, int threads) {
  std::vector<gem16::fp8::QuantizedToken> acts(tokens);
  for (uint64_t t = 0; t < tokens; ++t) {
    acts[t].logical_elements = k;
    acts[t].scale = a_scales[t];
    acts[t].values_e4m3fn.assign(a + t * k, a + (t + 1) * k);
  }
  std::atomic<int> status{0};
  parallel_for(rows, threads, [&](uint64_t r) {
    std::span<const uint8_t> wr(w + r * k, k);
    for (uint64_t t = 0; t < tokens; ++t) {
      auto d = gem16::fp8::ReferenceDotProduct(acts[t], wr, w_scales_bf16[r]);
      if (!d.ok()) {
        status = static_cast<int>(d.status().code());
        return;
      }
      out[t * rows + r] = d.value();
    }
  });
  return status.load();
}

// gem16::layer::RmsNorm (binary64 accumulation, fp32 result, no bf16 boundary); weight may be null.
int ref_rmsnorm(const float* x, const float* weight, uint64_t tokens, uint64_t k, float eps, float* out) {
  auto r = gem16::layer::RmsNorm(std::span<const float>(x, tokens * k),
                                 weight ? std::span<const float>(weight, k) : std::span<const float>(), tokens, k, eps);
  if (!r.ok()) return static_cast<int>(r.status().code());
  std::copy(r.value().begin(), r.value().end(), out);
  return 0;
}

}  // extern "C"
