// C++ mirror of the gpurs host surface for the matrix-multiply path, header-only, over the C ABI of
// include/gpurs_b200.h.  Names follow the reference so that its examples port line by line:
//
//   gpurs::Gpu gpu(0);                           Gpu::new(0)                 crates/gpurs/src/host/context.rs:69
//   auto stream = gpu.stream();                  gpu.stream()                context.rs:125
//   auto a = gpu.upload(host_vector);            gpu.upload(&host)           context.rs:132
//   auto c = gpu.zeros<float>(n);                gpu.zeros::<f32>(n)         context.rs:151
//   gpurs::matmul(stream, a, b, c, {m, n, k});   the launcher                crates/macros/src/launcher.rs:110-223
//   auto host = c.download();                    output.download()           crates/gpurs/src/host/memory/buffer.rs:251-271
//
// Where the reference returns `Result<T>`, these functions throw gpurs::Error carrying the same fields as
// `driver::Error` (crates/driver/src/error.rs:8-16).  Handles are move-only and belong to one host thread.
#pragma once
#include "../../include/gpurs_b200.h"

#include <array>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace gpurs {

// 16-bit and 8-bit storage formats: bit patterns, as `Half(pub u16)` / `BFloat16(pub u16)` / `E4M3(pub u8)` in
// crates/gpurs/src/gpu/float16.rs:8-14 and float8.rs:12-14.
struct Half { uint16_t bits; };
struct BFloat16 { uint16_t bits; };
struct E4M3 { uint8_t bits; };

template <class T> struct Element;
template <> struct Element<Half> { static constexpr int code = GPURS_F16; };
template <> struct Element<BFloat16> { static constexpr int code = GPURS_BF16; };
template <> struct Element<E4M3> { static constexpr int code = GPURS_E4M3; };
template <> struct Element<float> { static constexpr int code = GPURS_F32; };
template <> struct Element<int8_t> { static constexpr int code = GPURS_I8; };
template <> struct Element<int32_t> { static constexpr int code = GPURS_I32; };

class Error : public std::runtime_error {
  public:
    int code;
    std::string operation, name, description;
    explicit Error(int code_) : std::runtime_error(message(code_)), code(code_) {
        const char *o = "", *n = "", *d = "";
        gpurs_last_error(&o, &n, &d);
        operation = o, name = n, description = d;
    }
    bool is_out_of_memory() const { return code == 2; }                       // error.rs:23-25
    bool is_device_timeout() const { return code == GPURS_E_DEVICE_TIMEOUT; }

  private:
    static std::string message(int code) {
        const char *o = "", *n = "", *d = "";
        gpurs_last_error(&o, &n, &d);
        return std::string("`") + o + "` failed: " + n + " (" + d + ", code " + std::to_string(code) + ")";
    }
};

inline void check(int code) {
    if (code != GPURS_OK) throw Error(code);
}

// `LaunchConfig` (crates/gpurs/src/host/stream.rs:28-52) plus the cluster dimension.
struct LaunchConfig {
    std::array<uint32_t, 3> grid{1, 1, 1}, block{1, 1, 1};
    uint32_t shared_bytes = 0;
    std::array<uint32_t, 3> cluster{1, 1, 1};
    LaunchConfig(std::array<uint32_t, 3> g, std::array<uint32_t, 3> b) : grid(g), block(b) {}
    LaunchConfig &with_shared(uint32_t bytes) { shared_bytes = bytes; return *this; }
    LaunchConfig &with_cluster(std::array<uint32_t, 3> c) { cluster = c; return *this; }
};

class Gpu;

class Event {
  public:
    Event(Event &&other) noexcept : handle_(std::exchange(other.handle_, nullptr)) {}
    Event(const Event &) = delete;
    ~Event() { gpurs_event_free(handle_); }
    void synchronize() const { check(gpurs_event_synchronize(handle_)); }
    // milliseconds from this event to `later` (`Event::elapsed`)
    float elapsed_ms(const Event &later) const {
        float ms = 0;
        check(gpurs_event_elapsed_ms(handle_, later.handle_, &ms));
        return ms;
    }

  private:
    friend class Stream;
    explicit Event(gpurs_event *handle) : handle_(handle) {}
    gpurs_event *handle_;
};

class Stream {
  public:
    Stream(Stream &&other) noexcept : handle_(std::exchange(other.handle_, nullptr)) {}
    Stream(const Stream &) = delete;
    ~Stream() { gpurs_stream_free(handle_); }
    void synchronize() const { check(gpurs_stream_synchronize(handle_)); }
    Event record_timed() const {
        gpurs_event *event = nullptr;
        check(gpurs_event_record_timed(handle_, &event));
        return Event(event);
    }
    gpurs_stream *raw() const { return handle_; }

  private:
    friend class Gpu;
    explicit Stream(gpurs_stream *handle) : handle_(handle) {}
    gpurs_stream *handle_;
};

// A typed device allocation: the `DeviceSlice` / `DeviceSliceMut` of the reference (host/memory/buffer.rs:23-83).
template <class T>
class DeviceBuffer {
  public:
    DeviceBuffer(DeviceBuffer &&other) noexcept
        : gpu_(other.gpu_), pointer_(std::exchange(other.pointer_, 0)), length_(other.length_), owned_(other.owned_) {}
    DeviceBuffer(const DeviceBuffer &) = delete;
    ~DeviceBuffer() {
        if (owned_ && pointer_) gpurs_free(gpu_, pointer_);
    }
    size_t len() const { return length_; }
    gpurs_device_ptr address() const { return pointer_; }
    std::vector<T> download() const {
        std::vector<T> host(length_);
        check(gpurs_download(gpu_, pointer_, host.data(), length_ * sizeof(T)));
        return host;
    }

  private:
    friend class Gpu;
    DeviceBuffer(gpurs_gpu *gpu, gpurs_device_ptr pointer, size_t length, bool owned) : gpu_(gpu), pointer_(pointer), length_(length), owned_(owned) {}
    gpurs_gpu *gpu_;
    gpurs_device_ptr pointer_;
    size_t length_;
    bool owned_;
};

class Gpu {
  public:
    explicit Gpu(int ordinal) { check(gpurs_gpu_new(ordinal, &handle_)); }
    Gpu(const Gpu &) = delete;
    ~Gpu() { gpurs_gpu_free(handle_); }
    Stream stream() const {
        gpurs_stream *stream = nullptr;
        check(gpurs_stream_new(handle_, &stream));
        return Stream(stream);
    }
    template <class T> DeviceBuffer<T> upload(const std::vector<T> &host) const {
        gpurs_device_ptr pointer = 0;
        check(gpurs_upload(handle_, host.data(), host.size() * sizeof(T), &pointer));
        return DeviceBuffer<T>(handle_, pointer, host.size(), true);
    }
    template <class T> DeviceBuffer<T> zeros(size_t length) const {
        gpurs_device_ptr pointer = 0;
        check(gpurs_zeros(handle_, length * sizeof(T), &pointer));
        return DeviceBuffer<T>(handle_, pointer, length, true);
    }
    // `Gpu::import_allocation` (crates/gpurs/src/raw/allocation.rs:54-74): memory owned by someone else
    template <class T> DeviceBuffer<T> import_allocation(gpurs_device_ptr pointer, size_t length) const {
        return DeviceBuffer<T>(handle_, pointer, length, false);
    }
    int multiprocessors() const {
        int major, minor, count;
        size_t bytes;
        check(gpurs_gpu_properties(handle_, &major, &minor, &count, &bytes));
        return count;
    }
    gpurs_gpu *raw() const { return handle_; }

  private:
    gpurs_gpu *handle_ = nullptr;
};

struct MatmulOptions {
    uint64_t lda = 0, ldb = 0, ldc = 0;   // row pitches in elements, 0 = contiguous
    int algorithm = GPURS_ALGO_AUTO;
    int precision = GPURS_PRECISION_DEFAULT;
    gpurs_device_ptr scale_a = 0, scale_b = 0, metadata = 0;
    bool b_row_major = false;                                        // B given as k x n
    gpurs_device_ptr bias = 0, row_scale = 0, column_scale = 0;      // epilogue: acc * alpha * row_scale[r] * column_scale[c] + bias[c]
    float alpha = 0.0f;                                              // 0 = 1
};

// C[m, n] = sum_k A[m, k] * B[n, k]; shape = {m, n, k}.  A is m x k, B the n x k "right_transposed" operand of
// the reference's examples (examples/blackwell/examples/blackwell_matrix.rs:32-36), C m x n.  Validates, enqueues
// one kernel on `stream`, does not wait.
template <class A, class C>
void matmul(const Stream &stream, const DeviceBuffer<A> &a, const DeviceBuffer<A> &b, DeviceBuffer<C> &c, std::array<size_t, 3> shape,
            const MatmulOptions &options = {}) {
    gpurs_matmul_desc desc{};
    desc.a_type = Element<A>::code;
    desc.c_type = Element<C>::code;
    desc.m = shape[0], desc.n = shape[1], desc.k = shape[2];
    desc.lda = options.lda, desc.ldb = options.ldb, desc.ldc = options.ldc;
    desc.a_len = a.len(), desc.b_len = b.len(), desc.c_len = c.len();
    desc.algorithm = options.algorithm;
    desc.precision = options.precision;
    desc.scale_a = options.scale_a, desc.scale_b = options.scale_b, desc.metadata = options.metadata;
    desc.b_row_major = options.b_row_major ? 1 : 0;
    desc.bias = options.bias, desc.row_scale = options.row_scale, desc.column_scale = options.column_scale, desc.alpha = options.alpha;
    check(gpurs_matmul(stream.raw(), &desc, a.address(), b.address(), c.address()));
}

// The same product with operands and result in host memory (page-locked for the copies to overlap), staged through the
// device buffers: the example's upload / upload / launch / download as one call that overlaps the three.  Does not
// wait: synchronise `stream` before reading `host_c`.
template <class A, class C>
void matmul_host(const Stream &stream, const A *host_a, const A *host_b, C *host_c, DeviceBuffer<A> &a, DeviceBuffer<A> &b, DeviceBuffer<C> &c,
                 std::array<size_t, 3> shape, const MatmulOptions &options = {}) {
    gpurs_matmul_desc desc{};
    desc.a_type = Element<A>::code;
    desc.c_type = Element<C>::code;
    desc.m = shape[0], desc.n = shape[1], desc.k = shape[2];
    desc.lda = options.lda, desc.ldb = options.ldb, desc.ldc = options.ldc;
    desc.algorithm = options.algorithm;
    desc.precision = options.precision;
    desc.scale_a = options.scale_a, desc.scale_b = options.scale_b;
    desc.b_row_major = options.b_row_major ? 1 : 0;
    desc.bias = options.bias, desc.row_scale = options.row_scale, desc.column_scale = options.column_scale, desc.alpha = options.alpha;
    check(gpurs_matmul_host(stream.raw(), &desc, host_a, host_b, host_c, a.address(), b.address(), c.address()));
}

// output[r] = input[routes[r]] * weight[e]^T for offsets[e] <= r < offsets[e + 1]: the grouped (mixture-of-experts) product
// of the reference's `experts` example (examples/ada/examples/grouped_matrix.rs:30-60).
template <class A, class C>
void matmul_grouped(const Stream &stream, const DeviceBuffer<A> &input, const DeviceBuffer<uint32_t> &routes, const DeviceBuffer<uint32_t> &offsets,
                    const DeviceBuffer<A> &weight, DeviceBuffer<C> &output, size_t rows, size_t tokens, size_t n, size_t k, size_t experts) {
    gpurs_grouped_desc desc{};
    desc.a_type = Element<A>::code;
    desc.c_type = Element<C>::code;
    desc.rows = rows, desc.tokens = tokens, desc.n = n, desc.k = k, desc.experts = experts;
    check(gpurs_matmul_grouped(stream.raw(), &desc, input.address(), routes.address(), offsets.address(), weight.address(), output.address()));
}

// A recorded sequence of the calls above (`Graph` / `GraphExec`, crates/gpurs/src/host/graph/capture.rs:99-149, exec.rs:15-72).
class Graph {
  public:
    Graph(Graph &&other) noexcept : handle_(std::exchange(other.handle_, nullptr)) {}
    Graph(const Graph &) = delete;
    ~Graph() { gpurs_graph_free(handle_); }
    // Enqueues one replay of the whole recording on `stream`; does not wait.
    void launch(const Stream &stream) const { check(gpurs_graph_launch(handle_, stream.raw())); }

  private:
    template <class F> friend Graph capture(const Stream &stream, F &&record);
    explicit Graph(gpurs_graph *handle) : handle_(handle) {}
    gpurs_graph *handle_;
};

// `stream.capture(|capture| { ... })`: runs `record(stream)` with the stream recording instead of executing.
template <class F>
Graph capture(const Stream &stream, F &&record) {
    check(gpurs_stream_capture_begin(stream.raw()));
    gpurs_graph *handle = nullptr;
    try {
        record(stream);
    } catch (...) {
        if (gpurs_stream_capture_end(stream.raw(), &handle) == GPURS_OK) gpurs_graph_free(handle);
        throw;
    }
    check(gpurs_stream_capture_end(stream.raw(), &handle));
    return Graph(handle);
}

}  // namespace gpurs
