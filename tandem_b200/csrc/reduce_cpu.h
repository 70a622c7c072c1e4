// Element-wise arithmetic on host buffers for the CPU collectives: copy with an
// optional divide (gradient averaging divides every operand before it is
// summed, as torch DDP does; tandem/comm.py:336-339) and dst += src.  16-bit
// floats add in fp32 and round to nearest-even once per addition, the result
// ATen's CPU kernels give, so a sum folded in a fixed order is reproducible.
#pragma once

#include <cstdint>
#include <cstring>
#include <stdexcept>

namespace tb {

enum class DType : int { F32 = 0, F64 = 1, BF16 = 2, F16 = 3, I64 = 4, I32 = 5, I16 = 6, I8 = 7, U8 = 8 };

inline std::size_t dtype_size(DType d) {
  switch (d) {
    case DType::F32: case DType::I32: return 4;
    case DType::F64: case DType::I64: return 8;
    case DType::BF16: case DType::F16: case DType::I16: return 2;
    case DType::I8: case DType::U8: return 1;
  }
  throw std::invalid_argument("unknown dtype code");
}

inline bool dtype_is_float(DType d) { return d == DType::F32 || d == DType::F64 || d == DType::BF16 || d == DType::F16; }

struct bf16_t {
  std::uint16_t bits;
};
inline float to_float(bf16_t v) {
  std::uint32_t u = static_cast<std::uint32_t>(v.bits) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline bf16_t bf16_from(float f) {
  std::uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return bf16_t{static_cast<std::uint16_t>((u >> 16) | 0x0040u)};  // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1u);  // round to nearest, ties to even
  return bf16_t{static_cast<std::uint16_t>(u >> 16)};
}

template <class T>
struct Arith {
  static T add(T a, T b) { return static_cast<T>(a + b); }
  static T div(T a, int n) { return static_cast<T>(a / static_cast<T>(n)); }
};
template <>
struct Arith<bf16_t> {
  static bf16_t add(bf16_t a, bf16_t b) { return bf16_from(to_float(a) + to_float(b)); }
  static bf16_t div(bf16_t a, int n) { return bf16_from(to_float(a) / static_cast<float>(n)); }
};
template <>
struct Arith<_Float16> {
  static _Float16 add(_Float16 a, _Float16 b) { return static_cast<_Float16>(static_cast<float>(a) + static_cast<float>(b)); }
  static _Float16 div(_Float16 a, int n) { return static_cast<_Float16>(static_cast<float>(a) / static_cast<float>(n)); }
};

// The arrays these loops get never overlap (a tensor, this rank's slot, a peer's slot), which is what lets the
// compiler vectorise them; the one exception, add_own_t's copy == sum, is written as an in-place update.
template <class T>
void add_into_t(void* dst, const void* src, std::size_t n) {
  T* __restrict d = static_cast<T*>(dst);
  const T* __restrict s = static_cast<const T*>(src);
  for (std::size_t i = 0; i < n; ++i) d[i] = Arith<T>::add(d[i], s[i]);
}

template <class T>
void copy_div_t(void* dst, const void* src, std::size_t n, int divisor) {
  T* __restrict d = static_cast<T*>(dst);
  const T* __restrict s = static_cast<const T*>(src);
  for (std::size_t i = 0; i < n; ++i) d[i] = Arith<T>::div(s[i], divisor);
}

// dst[i] = a[i] + b[i]
template <class T>
void add2_t(void* dst, const void* a, const void* b, std::size_t n) {
  T* __restrict d = static_cast<T*>(dst);
  const T* __restrict x = static_cast<const T*>(a);
  const T* __restrict y = static_cast<const T*>(b);
  for (std::size_t i = 0; i < n; ++i) d[i] = Arith<T>::add(x[i], y[i]);
}

// own[i] = sum[i] + own[i] / divisor (divisor 0: no division); the result also goes to copy[i] when copy is given.
// copy is either a separate array or `sum` itself.
template <class T>
void add_own_t(void* own, void* copy, const void* sum, std::size_t n, int divisor) {
  T* __restrict o = static_cast<T*>(own);
  if (copy == nullptr) {
    const T* __restrict s = static_cast<const T*>(sum);
    if (divisor) for (std::size_t i = 0; i < n; ++i) o[i] = Arith<T>::add(s[i], Arith<T>::div(o[i], divisor));
    else for (std::size_t i = 0; i < n; ++i) o[i] = Arith<T>::add(s[i], o[i]);
  } else if (copy == sum) {
    T* __restrict s = static_cast<T*>(copy);
    if (divisor) for (std::size_t i = 0; i < n; ++i) o[i] = s[i] = Arith<T>::add(s[i], Arith<T>::div(o[i], divisor));
    else for (std::size_t i = 0; i < n; ++i) o[i] = s[i] = Arith<T>::add(s[i], o[i]);
  } else {
    T* __restrict c = static_cast<T*>(copy);
    const T* __restrict s = static_cast<const T*>(sum);
    if (divisor) for (std::size_t i = 0; i < n; ++i) o[i] = c[i] = Arith<T>::add(s[i], Arith<T>::div(o[i], divisor));
    else for (std::size_t i = 0; i < n; ++i) o[i] = c[i] = Arith<T>::add(s[i], o[i]);
  }
}

template <class F>
auto by_dtype(DType d, F&& f) {
  switch (d) {
    case DType::F32: return f(float{});
    case DType::F64: return f(double{});
    case DType::BF16: return f(bf16_t{});
    case DType::F16: return f(_Float16{});
    case DType::I64: return f(std::int64_t{});
    case DType::I32: return f(std::int32_t{});
    case DType::I16: return f(std::int16_t{});
    case DType::I8: return f(std::int8_t{});
    case DType::U8: return f(std::uint8_t{});
  }
  throw std::invalid_argument("unknown dtype code");
}

// dst[i] += src[i]
inline void add_into(void* dst, const void* src, std::size_t n, DType d) {
  by_dtype(d, [&](auto tag) { add_into_t<decltype(tag)>(dst, src, n); });
}

// dst[i] = a[i] + b[i]
inline void add2(void* dst, const void* a, const void* b, std::size_t n, DType d) {
  by_dtype(d, [&](auto tag) { add2_t<decltype(tag)>(dst, a, b, n); });
}

// own[i] = sum[i] + own[i] / divisor, also stored to copy[i] if copy != nullptr (see add_own_t)
inline void add_own(void* own, void* copy, const void* sum, std::size_t n, DType d, int divisor) {
  by_dtype(d, [&](auto tag) { add_own_t<decltype(tag)>(own, copy, sum, n, divisor); });
}

// dst[i] = src[i] / divisor (divisor 0: plain copy)
inline void copy_in(void* dst, const void* src, std::size_t n, DType d, int divisor) {
  if (divisor == 0) {
    if (n) std::memcpy(dst, src, n * dtype_size(d));
    return;
  }
  if (!dtype_is_float(d)) throw std::invalid_argument("avg needs a floating-point tensor");
  by_dtype(d, [&](auto tag) { copy_div_t<decltype(tag)>(dst, src, n, divisor); });
}

}  // namespace tb
