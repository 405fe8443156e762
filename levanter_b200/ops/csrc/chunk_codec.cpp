// Host-side chunk codec for zarr arrays (checkpoints and the token cache): zstd compression and
// decompression of many chunks in parallel on a thread pool.
//
// The reference delegates this to TensorStore (C++), reached through
// src/levanter/tensorstore_serialization.py:36-88.  libzstd is located at run time with dlopen, so
// the library builds without zstd headers; when it is missing the entry points return kErrNoZstd
// and callers store chunks uncompressed ("compressor": null), which every zarr reader accepts.
#include <dlfcn.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <mutex>
#include <thread>
#include <vector>

namespace {

constexpr int kOk = 0;
constexpr int kErrNoZstd = -10;
constexpr int kErrCodec = -11;
constexpr int kErrTooSmall = -12;

typedef size_t (*compress_fn)(void*, size_t, const void*, size_t, int);
typedef size_t (*decompress_fn)(void*, size_t, const void*, size_t);
typedef size_t (*bound_fn)(size_t);
typedef unsigned (*iserr_fn)(size_t);
typedef unsigned long long (*fcs_fn)(const void*, size_t);

struct Zstd {
  compress_fn compress = nullptr;
  decompress_fn decompress = nullptr;
  bound_fn bound = nullptr;
  iserr_fn is_error = nullptr;
  fcs_fn frame_content_size = nullptr;
  bool ok = false;
};

Zstd& zstd() {
  static Zstd z;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libzstd.so.1", "libzstd.so"};
    void* h = nullptr;
    for (const char* n : names) {
      h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (h) break;
    }
    if (!h) return;
    z.compress = reinterpret_cast<compress_fn>(dlsym(h, "ZSTD_compress"));
    z.decompress = reinterpret_cast<decompress_fn>(dlsym(h, "ZSTD_decompress"));
    z.bound = reinterpret_cast<bound_fn>(dlsym(h, "ZSTD_compressBound"));
    z.is_error = reinterpret_cast<iserr_fn>(dlsym(h, "ZSTD_isError"));
    z.frame_content_size = reinterpret_cast<fcs_fn>(dlsym(h, "ZSTD_getFrameContentSize"));
    z.ok = z.compress && z.decompress && z.bound && z.is_error && z.frame_content_size;
  });
  return z;
}

template <typename F>
void parallel_for(int n, int threads, F f) {
  if (threads <= 1 || n <= 1) {
    for (int i = 0; i < n; ++i) f(i);
    return;
  }
  if (threads > n) threads = n;
  std::atomic<int> next(0);
  std::vector<std::thread> pool;
  pool.reserve(threads);
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([&] {
      for (;;) {
        int i = next.fetch_add(1);
        if (i >= n) return;
        f(i);
      }
    });
  for (auto& th : pool) th.join();
}

}  // namespace

extern "C" int lvb_zstd_available() { return zstd().ok ? 1 : 0; }

extern "C" long long lvb_zstd_bound(long long n) {
  Zstd& z = zstd();
  if (!z.ok) return kErrNoZstd;
  return static_cast<long long>(z.bound(static_cast<size_t>(n)));
}

// Compress n chunks.  src[i]/src_len[i] -> dst[i] (capacity dst_cap[i]); out_len[i] receives the
// compressed size.  Returns 0 or the first error.
extern "C" int lvb_zstd_compress_many(int n, const void* const* src, const long long* src_len, void* const* dst,
                                      const long long* dst_cap, long long* out_len, int level, int threads) {
  Zstd& z = zstd();
  if (!z.ok) return kErrNoZstd;
  std::atomic<int> err(kOk);
  parallel_for(n, threads, [&](int i) {
    size_t r = z.compress(dst[i], static_cast<size_t>(dst_cap[i]), src[i], static_cast<size_t>(src_len[i]), level);
    if (z.is_error(r)) {
      err.store(kErrCodec);
      out_len[i] = -1;
    } else {
      out_len[i] = static_cast<long long>(r);
    }
  });
  return err.load();
}

// Size of the decoded frame stored in src (or a negative value when unknown).
extern "C" long long lvb_zstd_frame_size(const void* src, long long n) {
  Zstd& z = zstd();
  if (!z.ok) return kErrNoZstd;
  unsigned long long r = z.frame_content_size(src, static_cast<size_t>(n));
  if (r == static_cast<unsigned long long>(-1) || r == static_cast<unsigned long long>(-2)) return -1;
  return static_cast<long long>(r);
}

extern "C" int lvb_zstd_decompress_many(int n, const void* const* src, const long long* src_len, void* const* dst,
                                        const long long* dst_cap, long long* out_len, int threads) {
  Zstd& z = zstd();
  if (!z.ok) return kErrNoZstd;
  std::atomic<int> err(kOk);
  parallel_for(n, threads, [&](int i) {
    size_t r = z.decompress(dst[i], static_cast<size_t>(dst_cap[i]), src[i], static_cast<size_t>(src_len[i]));
    if (z.is_error(r)) {
      err.store(kErrCodec);
      out_len[i] = -1;
    } else {
      out_len[i] = static_cast<long long>(r);
    }
  });
  return err.load();
}
