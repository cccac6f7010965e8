// Parameter / optimizer-state checkpoints.  (The reference has no serialisation at all: a trained SNetwork
// lives and dies with its process.)
//
// File layout, little-endian:
//   char[8]  "FMLCKPT1"
//   u64      step            caller-defined counter (the optimizer's t)
//   u32      n_entries
//   per entry:  u32 name_len, name bytes, u64 n_floats, u32 crc32 (IEEE, of the payload bytes)
//   payloads in entry order, fp32
//
// Device buffers are staged through two pinned 16 MiB chunks: while chunk k is written to (or read from) the
// file, chunk k+1 is already crossing PCIe on a copy lane.  The file is written to "<path>.tmp" and renamed,
// so a crash never leaves a half-written checkpoint under the final name.
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include <fcntl.h>
#include <unistd.h>

#include "common.cuh"

namespace {

constexpr size_t CHUNK_FLOATS = 4u << 20;  // 16 MiB

uint32_t crc_table[256];
bool crc_ready = false;
void crc_init() {
  if (crc_ready) return;
  for (uint32_t i = 0; i < 256; i++) {
    uint32_t c = i;
    for (int k = 0; k < 8; k++) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
    crc_table[i] = c;
  }
  crc_ready = true;
}
uint32_t crc_update(uint32_t crc, const void* data, size_t n) {
  const unsigned char* p = static_cast<const unsigned char*>(data);
  crc = ~crc;
  for (size_t i = 0; i < n; i++) crc = crc_table[(crc ^ p[i]) & 0xFF] ^ (crc >> 8);
  return ~crc;
}

struct Staging {
  float* buf[2] = {nullptr, nullptr};
  cudaEvent_t ev[2] = {nullptr, nullptr};
  ~Staging() {
    for (int i = 0; i < 2; i++) {
      if (buf[i]) cudaFreeHost(buf[i]);
      if (ev[i]) cudaEventDestroy(ev[i]);
    }
  }
  bool init() {
    for (int i = 0; i < 2; i++) {
      if (cudaHostAlloc(reinterpret_cast<void**>(&buf[i]), CHUNK_FLOATS * 4, cudaHostAllocDefault) != cudaSuccess) return false;
      if (cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming) != cudaSuccess) return false;
    }
    return true;
  }
};

struct File {
  FILE* f = nullptr;
  std::string unlink_on_failure;   // a partly written temporary is removed unless the save completed
  ~File() {
    if (f) std::fclose(f);
    if (!unlink_on_failure.empty()) std::remove(unlink_on_failure.c_str());
  }
};

// flush a directory entry (the rename) to stable storage
void sync_parent_dir(const std::string& path) {
  const size_t slash = path.find_last_of('/');
  const std::string dir = slash == std::string::npos ? "." : (slash == 0 ? "/" : path.substr(0, slash));
  const int fd = ::open(dir.c_str(), O_RDONLY | O_DIRECTORY);
  if (fd >= 0) {
    ::fsync(fd);
    ::close(fd);
  }
}

struct Entry { std::string name; uint64_t n; uint32_t crc; };

}  // namespace

extern "C" {

int32_t fml_checkpoint_save(fml_ctx* ctx, const char* path, int64_t step, int32_t n, const char* const* names,
                            const float* const* bufs, const int64_t* sizes) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, path && n >= 0 && (n == 0 || (names && bufs && sizes)), "fml_checkpoint_save: bad arguments");
  for (int i = 0; i < n; i++)
    FML_REQUIRE(ctx, names[i] && bufs[i] && sizes[i] > 0 && std::strlen(names[i]) < 4096, "fml_checkpoint_save: bad entry");
  crc_init();
  Staging st;
  if (!st.init()) return fml_fail(ctx, FML_ERR_OOM, "fml_checkpoint_save: pinned staging allocation failed");
  cudaStream_t lane;
  int32_t rc = fml_any_stream(ctx, 1, &lane);
  if (rc) return rc;
  // the copy lane must see everything queued on the main stream so far
  FML_CUDA(ctx, cudaEventRecord(st.ev[0], ctx->stream));
  FML_CUDA(ctx, cudaStreamWaitEvent(lane, st.ev[0], 0));

  const std::string tmp = std::string(path) + ".tmp";
  File out;
  out.f = std::fopen(tmp.c_str(), "wb");
  if (!out.f) return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_save: cannot open " + tmp);
  out.unlink_on_failure = tmp;
  // header with zero CRCs first; rewritten once the payload has passed through the host
  std::vector<uint32_t> crcs(n, 0);
  auto write_header = [&]() -> bool {
    const uint64_t step_u = (uint64_t)step;
    const uint32_t cnt = (uint32_t)n;
    bool ok = std::fwrite("FMLCKPT1", 1, 8, out.f) == 8 && std::fwrite(&step_u, 8, 1, out.f) == 1 && std::fwrite(&cnt, 4, 1, out.f) == 1;
    for (int i = 0; i < n && ok; i++) {
      const uint32_t len = (uint32_t)std::strlen(names[i]);
      const uint64_t cntf = (uint64_t)sizes[i];
      ok = std::fwrite(&len, 4, 1, out.f) == 1 && std::fwrite(names[i], 1, len, out.f) == len &&
           std::fwrite(&cntf, 8, 1, out.f) == 1 && std::fwrite(&crcs[i], 4, 1, out.f) == 1;
    }
    return ok;
  };
  if (!write_header()) return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_save: write failed");
  for (int i = 0; i < n; i++) {
    const size_t total = (size_t)sizes[i];
    const size_t chunks = (total + CHUNK_FLOATS - 1) / CHUNK_FLOATS;
    auto issue = [&](size_t k) -> cudaError_t {
      const size_t off = k * CHUNK_FLOATS, cnt = std::min(CHUNK_FLOATS, total - off);
      cudaError_t e = cudaMemcpyAsync(st.buf[k & 1], bufs[i] + off, cnt * 4, cudaMemcpyDeviceToHost, lane);
      return e != cudaSuccess ? e : cudaEventRecord(st.ev[k & 1], lane);
    };
    FML_CUDA(ctx, issue(0));
    for (size_t k = 0; k < chunks; k++) {
      if (k + 1 < chunks) FML_CUDA(ctx, issue(k + 1));
      FML_CUDA(ctx, cudaEventSynchronize(st.ev[k & 1]));
      const size_t cnt = std::min(CHUNK_FLOATS, total - k * CHUNK_FLOATS);
      crcs[i] = crc_update(crcs[i], st.buf[k & 1], cnt * 4);
      if (std::fwrite(st.buf[k & 1], 4, cnt, out.f) != cnt) return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_save: write failed");
    }
  }
  // the bytes reach stable storage before the file takes its final name, and the rename itself is made durable:
  // after a crash the name holds either the old complete file or the new complete file
  if (std::fseek(out.f, 0, SEEK_SET) != 0 || !write_header() || std::fflush(out.f) != 0 || ::fsync(::fileno(out.f)) != 0)
    return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_save: write failed");
  std::fclose(out.f);
  out.f = nullptr;
  if (std::rename(tmp.c_str(), path) != 0) return fml_fail(ctx, FML_ERR_INVALID, std::string("fml_checkpoint_save: cannot rename to ") + path);
  out.unlink_on_failure.clear();
  sync_parent_dir(path);
  return FML_OK;
}

int32_t fml_checkpoint_load(fml_ctx* ctx, const char* path, int64_t* step, int32_t n, const char* const* names,
                            float* const* bufs, const int64_t* sizes) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, path && n >= 0 && (n == 0 || (names && bufs && sizes)), "fml_checkpoint_load: bad arguments");
  crc_init();
  File in;
  in.f = std::fopen(path, "rb");
  if (!in.f) return fml_fail(ctx, FML_ERR_INVALID, std::string("fml_checkpoint_load: cannot open ") + path);
  char magic[8];
  uint64_t step_u = 0;
  uint32_t cnt = 0;
  if (std::fread(magic, 1, 8, in.f) != 8 || std::memcmp(magic, "FMLCKPT1", 8) != 0)
    return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_load: not a checkpoint file");
  if (std::fread(&step_u, 8, 1, in.f) != 1 || std::fread(&cnt, 4, 1, in.f) != 1 || cnt > (1u << 20))
    return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_load: truncated header");
  std::vector<Entry> entries(cnt);
  for (Entry& e : entries) {
    uint32_t len = 0;
    if (std::fread(&len, 4, 1, in.f) != 1 || len >= 4096) return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_load: truncated header");
    e.name.resize(len);
    if ((len && std::fread(&e.name[0], 1, len, in.f) != len) || std::fread(&e.n, 8, 1, in.f) != 1 || std::fread(&e.crc, 4, 1, in.f) != 1)
      return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_load: truncated header");
  }
  const long payload0 = std::ftell(in.f);
  // every requested name must exist with the requested size before anything is overwritten
  std::vector<int> where(n, -1);
  for (int i = 0; i < n; i++) {
    FML_REQUIRE(ctx, names[i] && bufs[i] && sizes[i] > 0, "fml_checkpoint_load: bad entry");
    for (uint32_t j = 0; j < cnt; j++)
      if (entries[j].name == names[i]) where[i] = (int)j;
    if (where[i] < 0) return fml_fail(ctx, FML_ERR_INVALID, std::string("fml_checkpoint_load: no entry named ") + names[i]);
    if (entries[where[i]].n != (uint64_t)sizes[i])
      return fml_fail(ctx, FML_ERR_INVALID, std::string("fml_checkpoint_load: size mismatch for ") + names[i]);
  }
  Staging st;
  if (!st.init()) return fml_fail(ctx, FML_ERR_OOM, "fml_checkpoint_load: pinned staging allocation failed");
  cudaStream_t lane;
  int32_t rc = fml_any_stream(ctx, 1, &lane);
  if (rc) return rc;
  FML_CUDA(ctx, cudaEventRecord(st.ev[0], ctx->stream));
  FML_CUDA(ctx, cudaStreamWaitEvent(lane, st.ev[0], 0));
  FML_CUDA(ctx, cudaEventSynchronize(st.ev[0]));
  auto seek_to = [&](int entry) -> bool {
    uint64_t off_floats = 0;
    for (int j = 0; j < entry; j++) off_floats += entries[j].n;
    return std::fseek(in.f, payload0 + (long)(off_floats * 4), SEEK_SET) == 0;
  };
  // pass 1: checksums of every requested entry, before any device buffer is overwritten
  for (int i = 0; i < n; i++) {
    const Entry& e = entries[where[i]];
    if (!seek_to(where[i])) return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_load: seek failed");
    uint32_t crc = 0;
    for (size_t done = 0; done < e.n; done += CHUNK_FLOATS) {
      const size_t c = std::min<size_t>(CHUNK_FLOATS, e.n - done);
      if (std::fread(st.buf[0], 4, c, in.f) != c) return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_load: truncated payload");
      crc = crc_update(crc, st.buf[0], c * 4);
    }
    if (crc != e.crc) return fml_fail(ctx, FML_ERR_INVALID, std::string("fml_checkpoint_load: checksum mismatch in ") + names[i]);
  }
  // pass 2: file -> pinned chunk -> device, the read of chunk k+1 overlapping the copy of chunk k
  bool used[2] = {false, false};
  for (int i = 0; i < n; i++) {
    const Entry& e = entries[where[i]];
    if (!seek_to(where[i])) return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_load: seek failed");
    const size_t total = (size_t)e.n, chunks = (total + CHUNK_FLOATS - 1) / CHUNK_FLOATS;
    for (size_t k = 0; k < chunks; k++) {
      const int b = (int)(k & 1);
      if (used[b]) FML_CUDA(ctx, cudaEventSynchronize(st.ev[b]));  // the copy that last read this chunk has finished
      const size_t c = std::min(CHUNK_FLOATS, total - k * CHUNK_FLOATS);
      if (std::fread(st.buf[b], 4, c, in.f) != c) return fml_fail(ctx, FML_ERR_INVALID, "fml_checkpoint_load: truncated payload");
      FML_CUDA(ctx, cudaMemcpyAsync(bufs[i] + k * CHUNK_FLOATS, st.buf[b], c * 4, cudaMemcpyHostToDevice, lane));
      FML_CUDA(ctx, cudaEventRecord(st.ev[b], lane));
      used[b] = true;
    }
  }
  FML_CUDA(ctx, cudaStreamSynchronize(lane));
  // later work on the main stream sees the restored buffers
  FML_CUDA(ctx, cudaEventRecord(st.ev[0], lane));
  FML_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, st.ev[0], 0));
  FML_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (step) *step = (int64_t)step_u;
  return FML_OK;
}

}  // extern "C"
