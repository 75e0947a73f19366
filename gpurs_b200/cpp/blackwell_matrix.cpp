// The reference's Blackwell example (examples/blackwell/examples/blackwell_matrix.rs:58-83) and its shared
// harness (examples/matrix_benchmark.rs) on this library: the same inputs, the same 5 + 50 launch timing
// protocol, the same sampled fp64 check and the same printed line; the tile constants, tensor maps and launch
// geometry of the original disappear into `matmul`.
//
//   g++ -std=c++17 -O2 blackwell_matrix.cpp -o blackwell_matrix -L.. -lgpurs_b200 -Wl,-rpath,'$ORIGIN/..'
//   ./blackwell_matrix [size]
#include "gpurs.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

using gpurs::Half;

// f32 -> binary16 for the multiples of 1/16 in [-1, 1) the example uses (exact: no rounding case arises).
static Half half_from_exact(float value) {
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    const uint32_t sign = (bits >> 16) & 0x8000u, exponent = (bits >> 23) & 0xffu, mantissa = bits & 0x7fffffu;
    if (exponent == 0) return Half{uint16_t(sign)};
    return Half{uint16_t(sign | ((exponent - 112u) << 10) | (mantissa >> 13))};
}

static double half_to_f64(Half h) {
    const int exponent = (h.bits >> 10) & 0x1f, mantissa = h.bits & 0x3ff;
    const double magnitude = exponent == 0 ? std::ldexp(double(mantissa), -24) : std::ldexp(double(mantissa | 0x400), exponent - 25);
    return (h.bits & 0x8000) ? -magnitude : magnitude;
}

// matrix_benchmark.rs:5-14
static std::pair<std::vector<Half>, std::vector<Half>> inputs(size_t size) {
    std::vector<Half> left(size * size), right(size * size);
    for (size_t index = 0; index < size * size; index++) {
        left[index] = half_from_exact(float(index * 13 % 31) / 16.0f - 1.0f);
        right[index] = half_from_exact(float(index * 7 % 29) / 16.0f - 1.0f);
    }
    return {std::move(left), std::move(right)};
}

// matrix_benchmark.rs:16-27: 5 untimed launches, then 50 timed by the host clock, one synchronize per batch
template <class Launch>
static double measure(const gpurs::Stream &stream, Launch launch) {
    for (int i = 0; i < 5; i++) launch();
    stream.synchronize();
    const auto start = std::chrono::steady_clock::now();
    for (int i = 0; i < 50; i++) launch();
    stream.synchronize();
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count() / 50.0;
}

// matrix_benchmark.rs:29-58: sampled fp64 check, printed line, error bound 1e-2
static bool report(size_t size, double seconds, const std::vector<Half> &left, const std::vector<Half> &right, const std::vector<float> &product) {
    double error = 0.0;
    const size_t step = std::max<size_t>(size * size / 4093, 1);
    for (size_t index = 0; index < size * size; index += step) {
        const size_t row = index / size, column = index % size;
        double expected = 0.0;
        for (size_t depth = 0; depth < size; depth++) expected += half_to_f64(left[row * size + depth]) * half_to_f64(right[column * size + depth]);
        error = std::max(error, std::fabs(double(product[index]) - expected));
    }
    std::printf("%zux%zux%zu: %.3f ms, %.1f TFLOP/s, max abs error %.2e\n", size, size, size, seconds * 1e3,
                2.0 * double(size) * double(size) * double(size) / seconds / 1e12, error);
    return error < 1e-2;
}

int main(int argc, char **argv) {
    const size_t size = argc > 1 ? std::strtoull(argv[1], nullptr, 10) : 4096;
    try {
        gpurs::Gpu gpu(0);
        auto stream = gpu.stream();
        auto [left_host, right_host] = inputs(size);
        auto left = gpu.upload(left_host);
        auto right_transposed = gpu.upload(right_host);
        auto output = gpu.zeros<float>(size * size);
        const double seconds = measure(stream, [&] { gpurs::matmul(stream, left, right_transposed, output, {size, size, size}); });
        if (!report(size, seconds, left_host, right_host, output.download())) {
            std::fprintf(stderr, "the product differs from the reference\n");
            return 1;
        }
    } catch (const gpurs::Error &error) {
        std::fprintf(stderr, "%s\n", error.what());
        return 2;
    }
    return 0;
}
