// Host-side group quantiser of the converter: fp32 / bf16 / fp16 tensors -> INT4 asymmetric or INT8 symmetric groups,
// multi-threaded, bit-identical to zse_b200/format/quantize.py (rounding="nearest": double precision, round half to
// even, correctly rounded fp16 scales).  Role of the C helper the reference compiles with gcc at run time
// (zse-engine/zse_engine/format/fast_quant.py:24-226); here it is part of the ahead-of-time library.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

inline uint16_t f16_bits(double v) {
  _Float16 h = static_cast<_Float16>(v);
  uint16_t u;
  std::memcpy(&u, &h, 2);
  return u;
}

template <typename Fn>
void parallel_groups(int64_t n_groups, Fn fn) {
  unsigned hw = std::thread::hardware_concurrency();
  int n_threads = int(std::min<int64_t>(std::max(1u, std::min(hw, 32u)), (n_groups + 4095) / 4096));
  if (n_threads <= 1) {
    fn(0, n_groups);
    return;
  }
  std::vector<std::thread> pool;
  const int64_t per = (n_groups + n_threads - 1) / n_threads;
  for (int t = 0; t < n_threads; ++t) {
    const int64_t a = t * per, b = std::min(n_groups, a + per);
    if (a < b) pool.emplace_back(fn, a, b);
  }
  for (auto& th : pool) th.join();
}

}  // namespace

// values: n elements (fp32); groups run over the flattened tensor, the last one is zero padded.
// packed: ceil(n/gs)*gs/2 bytes, scales/zeros: ceil(n/gs) fp16 each.
extern "C" int zse_host_quantize_int4(const float* values, int64_t n, int group_size, uint8_t* packed,
                                      uint16_t* scales, uint16_t* zeros) {
  if (n < 0 || group_size <= 0 || group_size % 2) return -1;
  const int64_t n_groups = (n + group_size - 1) / group_size;
  parallel_groups(n_groups, [=](int64_t g0, int64_t g1) {
    std::vector<double> buf(group_size);
    for (int64_t g = g0; g < g1; ++g) {
      const int64_t base = g * group_size;
      const int valid = int(std::min<int64_t>(group_size, n - base));
      double lo = 1e300, hi = -1e300;
      for (int i = 0; i < group_size; ++i) {
        const double v = i < valid ? double(values[base + i]) : 0.0;
        buf[i] = v;
        lo = std::min(lo, v);
        hi = std::max(hi, v);
      }
      const double rng = hi - lo;
      const double scale = rng < 1e-10 ? 1.0 : rng / 15.0;
      const double inv = 1.0 / scale;
      uint8_t* out = packed + base / 2;
      for (int i = 0; i < group_size; i += 2) {
        int q0 = int(std::nearbyint((buf[i] - lo) * inv));
        int q1 = int(std::nearbyint((buf[i + 1] - lo) * inv));
        q0 = std::min(15, std::max(0, q0));
        q1 = std::min(15, std::max(0, q1));
        out[i / 2] = uint8_t(q0 | (q1 << 4));
      }
      scales[g] = f16_bits(scale);
      zeros[g] = f16_bits(lo);
    }
  });
  return 0;
}

// INT8 symmetric: scale = amax / 127 (1.0 for an all-zero group), q = rint(v * 127 / amax) in fp32 like the numpy path.
extern "C" int zse_host_quantize_int8(const float* values, int64_t n, int group_size, int8_t* q, uint16_t* scales) {
  if (n < 0 || group_size <= 0) return -1;
  const int64_t n_groups = (n + group_size - 1) / group_size;
  parallel_groups(n_groups, [=](int64_t g0, int64_t g1) {
    for (int64_t g = g0; g < g1; ++g) {
      const int64_t base = g * group_size;
      const int valid = int(std::min<int64_t>(group_size, n - base));
      float amax = 0.f;
      for (int i = 0; i < valid; ++i) amax = std::max(amax, std::fabs(values[base + i]));
      const bool ok = amax > 1e-10f;
      const float scale = ok ? amax / 127.0f : 1.0f;
      const float inv = ok ? 127.0f / amax : 0.0f;
      for (int i = 0; i < group_size; ++i) {
        const float v = i < valid ? values[base + i] * inv : 0.f;
        int r = int(std::nearbyintf(v));
        q[base + i] = int8_t(std::min(127, std::max(-128, r)));
      }
      scales[g] = f16_bits(double(scale));
    }
  });
  return 0;
}

extern "C" void zse_host_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t u = uint32_t(src[i]) << 16;
    std::memcpy(&dst[i], &u, 4);
  }
}

extern "C" void zse_host_f16_to_f32(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    _Float16 h;
    std::memcpy(&h, &src[i], 2);
    dst[i] = float(h);
  }
}

extern "C" void zse_host_f32_to_f16(const float* src, uint16_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = f16_bits(double(src[i]));
}
