// C++ port of the reference's FFI test (crates/hal-ffi/tests/test_ffi_mock.rs:48-157) on top of hal.hpp.
// usage: ffi_port <library.so> [expected-name]   -- exit code 0 = all checks passed.
// The same binary runs against the reference's own mock_npu.c build and against libsptorch_b200.so.
#include "../sptorch_b200/csrc/hal.hpp"
#include <cmath>
#include <cstdio>
#include <cstring>

using namespace sptorch_b200;
static int failures = 0;
#define CHECK(cond) do { if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); failures++; } } while (0)
static bool eq(const std::vector<float>& a, std::initializer_list<float> b) { return a == std::vector<float>(b); }

// crates/hal/src/lib.rs:674-700: pure host bookkeeping, needs no backend
static void kv_cache_metadata_tests() {
    KvCacheBufferSpec spec(DeviceId{"cuda", 0}, DType::BF16, 2, 4, 3, 8);                 // test_kv_cache_buffer_spec_layout_and_capacity
    CHECK(spec.elements_per_kind() == 2 * 4 * 3 * 8);
    CHECK(spec.total_elements() == 2 * 2 * 4 * 3 * 8);
    CHECK(spec.total_bytes() == 2 * 2 * 4 * 3 * 8 * 2);
    CHECK(spec.element_offset(1, 2, 1, 3) == (((4 + 2) * 3 + 1) * 8) + 3);
    bool threw = false;
    try { spec.element_offset(2, 0, 0, 0); } catch (const HalError&) { threw = true; }
    CHECK(threw);
    KvCacheWindowState w(3);                                                              // test_kv_cache_window_state_prefill_and_append
    size_t last = 99;
    CHECK(w.next_position() == 0 && !w.last_position(&last));
    w.prefill(5, 2);
    CHECK(w.window_start == 5 && w.cached_len == 2 && w.last_position(&last) && last == 6 && w.next_position() == 7);
    w.append(2);
    CHECK(w.window_start == 6 && w.cached_len == 3 && w.last_position(&last) && last == 8 && w.next_position() == 9);
    KvCacheWindowState v(3);                                                              // window part of test_cpu_kv_cache_buffer_tracks_capacity_and_window
    v.prefill(10, 3); v.append(1);
    KvCacheWindowState want(3); want.window_start = 11; want.cached_len = 3;
    CHECK(v == want);
}

int main(int argc, char** argv) {
    if (argc == 2 && std::string(argv[1]) == "--metadata") { kv_cache_metadata_tests(); std::printf(failures ? "FAILED %d\n" : "OK\n", failures); return failures ? 1 : 0; }
    if (argc < 2) { std::printf("usage: %s lib.so [name]\n", argv[0]); return 2; }
    std::shared_ptr<FfiBackend> be;
    try { be = FfiBackend::load(argv[1]); }
    catch (const HalError& e) { std::printf("LOAD_FAILED %s\n", e.what()); return 3; }
    std::vector<float> out;
    if (argc > 2) CHECK(be->name() == argv[2]);                                          // test_ffi_backend_name
    be->add_f32({1, 2, 3}, {4, 5, 6}, out); CHECK(eq(out, {5, 7, 9}));                   // test_ffi_add
    be->mul_f32({2, 3}, {4, 5}, out); CHECK(eq(out, {8, 15}));                           // test_ffi_mul
    be->neg_f32({1, -2, 3}, out); CHECK(eq(out, {-1, 2, -3}));                           // test_ffi_neg
    be->scale_f32({1, 2, 3}, 0.5f, out); CHECK(eq(out, {0.5f, 1.0f, 1.5f}));             // test_ffi_scale
    be->relu_f32({-1, 0, 2, -0.5f}, out); CHECK(eq(out, {0, 0, 2, 0}));                  // test_ffi_relu
    be->matmul_f32({1, 2, 3, 4, 5, 6}, {7, 8, 9, 10, 11, 12}, out, 2, 3, 2);             // test_ffi_matmul
    CHECK(eq(out, {58, 64, 139, 154}));
    be->softmax_f32({1, 2, 3}, out, 1, 3);                                               // test_ffi_softmax
    CHECK(std::fabs(out[0] + out[1] + out[2] - 1.0f) < 1e-6f && out[2] > out[1] && out[1] > out[0]);
    { std::vector<float> d{1, 2, 3, 4}; RawBuffer b = be->upload(d); CHECK(b.to_host() == d); }   // test_ffi_upload_download
    { std::vector<float> e, l; be->exp_f32({0, 1, 2}, e); be->log_f32(e, l);             // test_ffi_exp_log_roundtrip
      for (int i = 0; i < 3; i++) CHECK(std::fabs(l[i] - (float)i) < 1e-5f); }
    { uint32_t q = 99; bool on = false; be->synchronize();                               // test_ffi_query_runtime_optional_hook
      CHECK(be->query_runtime(&q, &on)); CHECK(q == 0 && on); }
    { std::vector<float> a{1, 2, 3, 4, 5, 6, 7, 8}, id{1, 0, 0, 1, 1, 0, 0, 1};           // hal/src/lib.rs:838-846
      be->batch_matmul_f32(a, id, out, 2, 2, 2, 2); CHECK(out == a); }
    be->gelu_f32({0, 1, -1}, out);                                                       // hal/src/lib.rs:804-812
    CHECK(std::fabs(out[0]) < 1e-6f && std::fabs(out[1] - 0.8413f) < 1e-3f && std::fabs(out[2] + 0.1587f) < 1e-3f);
    std::printf(failures ? "FAILED %d\n" : "OK\n", failures);
    return failures ? 1 : 0;
}
