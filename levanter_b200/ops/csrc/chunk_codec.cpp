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

// ---------------------------------------------------------------------------------------------------------------------
// Blosc (version 1 frames) decoder, LZ4 block decoder and CRC-32C: what it takes to read the token caches the reference
// writes (zarr v3 arrays whose shards hold blosc-compressed inner chunks followed by an index with a CRC-32C,
// src/levanter/store/jagged_array.py:605-635).  Decode only; this framework writes its own caches as zarr v2 + zstd.
//
// A blosc frame: 16-byte header {version, versionlz, flags, typesize, nbytes u32, blocksize u32, cbytes u32}; flags bit 0 =
// byte shuffle, bit 1 = stored uncompressed right after the header, bit 2 = bit shuffle (not decoded here), bit 4 = blocks
// are not split, bits 5-7 = compressor (0 blosclz, 1 lz4, 2 snappy, 3 zlib, 4 zstd; lz4 and zstd are decoded here).  Then
// one int32 offset per block, then the blocks.  A block that is split holds `typesize` streams (the bytes of equal
// significance of its elements after the shuffle), each prefixed by its compressed size; a stream whose compressed size
// equals its raw size is stored raw.  The last, shorter block is never split.
namespace {

constexpr int kErrBlosc = -13;

inline uint32_t rd32(const uint8_t* p) { return p[0] | (p[1] << 8) | (p[2] << 16) | (static_cast<uint32_t>(p[3]) << 24); }

long long lz4_block(const uint8_t* src, long long n, uint8_t* dst, long long cap) {
  const uint8_t* ip = src;
  const uint8_t* const iend = src + n;
  uint8_t* op = dst;
  uint8_t* const oend = dst + cap;
  while (ip < iend) {
    const unsigned token = *ip++;
    long long lit = token >> 4;
    if (lit == 15) {
      unsigned b;
      do {
        if (ip >= iend) return -1;
        b = *ip++;
        lit += b;
      } while (b == 255);
    }
    if (lit > iend - ip || lit > oend - op) return -1;
    for (long long i = 0; i < lit; ++i) op[i] = ip[i];
    ip += lit;
    op += lit;
    if (ip >= iend) break;  // the last sequence has no match part
    if (iend - ip < 2) return -1;
    const long long off = ip[0] | (ip[1] << 8);
    ip += 2;
    if (off == 0 || off > op - dst) return -1;
    long long len = token & 15;
    if (len == 15) {
      unsigned b;
      do {
        if (ip >= iend) return -1;
        b = *ip++;
        len += b;
      } while (b == 255);
    }
    len += 4;
    if (len > oend - op) return -1;
    const uint8_t* m = op - off;
    for (long long i = 0; i < len; ++i) op[i] = m[i];  // byte by byte: the match may overlap its own output
    op += len;
  }
  return op - dst;
}

long long blosc_frame(const uint8_t* src, long long srclen, uint8_t* dst, long long cap) {
  if (srclen < 16) return kErrBlosc;
  const unsigned flags = src[2];
  const int typesize = src[3];
  const long long nbytes = rd32(src + 4), blocksize = rd32(src + 8), cbytes = rd32(src + 12);
  if (cbytes > srclen || nbytes > cap || typesize <= 0) return kErrBlosc;
  if (nbytes == 0) return 0;
  if (flags & 0x2) {  // stored
    if (16 + nbytes > srclen) return kErrBlosc;
    for (long long i = 0; i < nbytes; ++i) dst[i] = src[16 + i];
    return nbytes;
  }
  if (flags & 0x4) return kErrBlosc;  // bit shuffle
  const int codec = (flags >> 5) & 7;
  if (codec != 1 && codec != 4) return kErrBlosc;
  if (codec == 4 && !zstd().ok) return kErrNoZstd;
  if (blocksize <= 0) return kErrBlosc;
  const bool shuffle = (flags & 0x1) && typesize > 1;
  const bool dont_split = (flags & 0x10) != 0;
  const long long nblocks = (nbytes + blocksize - 1) / blocksize;
  if (16 + 4 * nblocks > srclen) return kErrBlosc;
  std::vector<uint8_t> tmp(shuffle ? static_cast<size_t>(blocksize) : 0);
  for (long long blk = 0; blk < nblocks; ++blk) {
    const long long bsize = (blk == nblocks - 1 && nbytes % blocksize) ? nbytes % blocksize : blocksize;
    const bool leftover = bsize != blocksize;
    const long long start = rd32(src + 16 + 4 * blk);
    if (start < 16 + 4 * nblocks || start > srclen) return kErrBlosc;
    const uint8_t* ip = src + start;
    const int nsplits = (!dont_split && typesize <= 16 && blocksize / typesize >= 128 && !leftover) ? typesize : 1;
    const long long ne = bsize / nsplits;
    uint8_t* out = shuffle ? tmp.data() : dst + blk * blocksize;
    for (int s = 0; s < nsplits; ++s) {
      if (src + srclen - ip < 4) return kErrBlosc;
      const long long c = rd32(ip);
      ip += 4;
      if (c < 0 || c > src + srclen - ip) return kErrBlosc;
      if (c == ne) {
        for (long long i = 0; i < ne; ++i) out[s * ne + i] = ip[i];
      } else if (codec == 1) {
        if (lz4_block(ip, c, out + s * ne, ne) != ne) return kErrBlosc;
      } else {
        const size_t r = zstd().decompress(out + s * ne, static_cast<size_t>(ne), ip, static_cast<size_t>(c));
        if (zstd().is_error(r) || static_cast<long long>(r) != ne) return kErrBlosc;
      }
      ip += c;
    }
    if (shuffle) {
      // undo the byte shuffle of this block: byte j of element i sits at j * n + i; a tail shorter than an element is as is
      uint8_t* d = dst + blk * blocksize;
      const long long nel = bsize / typesize;
      for (long long i = 0; i < nel; ++i)
        for (int j = 0; j < typesize; ++j) d[i * typesize + j] = tmp[j * nel + i];
      for (long long i = nel * typesize; i < bsize; ++i) d[i] = tmp[i];
    }
  }
  return nbytes;
}

uint32_t crc32c_table[256];
std::once_flag crc_once;

}  // namespace

// Decoded size of a blosc frame (its header's nbytes), or a negative error.
extern "C" long long lvb_blosc_nbytes(const void* src, long long n) {
  if (n < 16) return kErrBlosc;
  return rd32(static_cast<const uint8_t*>(src) + 4);
}

// Decode n blosc frames in parallel; out_len[i] = decoded bytes or a negative error.  Returns 0 or the first error.
extern "C" int lvb_blosc_decompress_many(int n, const void* const* src, const long long* src_len, void* const* dst,
                                         const long long* dst_cap, long long* out_len, int threads) {
  std::atomic<int> err(kOk);
  parallel_for(n, threads, [&](int i) {
    const long long r = blosc_frame(static_cast<const uint8_t*>(src[i]), src_len[i], static_cast<uint8_t*>(dst[i]), dst_cap[i]);
    out_len[i] = r;
    if (r < 0) err.store(static_cast<int>(r));
  });
  return err.load();
}

// One raw LZ4 block (no frame): decoded bytes or -1.
extern "C" long long lvb_lz4_decompress_block(const void* src, long long n, void* dst, long long cap) {
  return lz4_block(static_cast<const uint8_t*>(src), n, static_cast<uint8_t*>(dst), cap);
}

// CRC-32C (Castagnoli, reflected polynomial 0x82F63B78), as stored after a zarr v3 shard index.
extern "C" unsigned lvb_crc32c(const void* data, long long n) {
  std::call_once(crc_once, [] {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (c >> 1) ^ 0x82F63B78u : c >> 1;
      crc32c_table[i] = c;
    }
  });
  uint32_t c = 0xFFFFFFFFu;
  const uint8_t* p = static_cast<const uint8_t*>(data);
  for (long long i = 0; i < n; ++i) c = crc32c_table[(c ^ p[i]) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}
