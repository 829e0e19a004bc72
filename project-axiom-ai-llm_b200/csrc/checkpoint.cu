// MoE block of the engine's checkpoint file: host-side save / probe / load, and the
// fp32 -> bf16 cast that rebuilds the working copy after a load.
//
// The engine writes `weights.axiom` as a 56-byte packed header ("AXIOM_V1", six u64:
// input and target element totals, weight count, bias count, vocabulary size,
// embedding dimension; core/include/config.hpp:41-55), then fp32 weights, bias and
// vocab x dim embeddings, then optionally a transformer block: u64 tag 0x5458464D,
// u64 dim, u64 ffn, four dim x dim and three dim x ffn fp32 matrices
// (core/src/training.cpp:283-392).  Its loader (core/src/ai.cpp:273-491) reads a u64
// after the embeddings, requires it to be that tag, reads the block and then stops,
// so anything after the transformer block is invisible to it.  That is where the MoE
// block goes; the format is described in include/axm_moe.h.  Same protocol as the
// engine's writer: refuse non-finite values, write `path`.tmp, rename over `path`.
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"

namespace axm {
namespace {

constexpr uint64_t kStockTag = 0x5458464DULL;  // the engine's transformer block
constexpr uint64_t kMoeTag = 0x4D4F4558ULL;    // this library's MoE block
constexpr uint64_t kMoeVersion = 1;
constexpr size_t kChunkFloats = 1u << 20;  // 4 MiB at a time

struct StockHeader {  // 56 bytes, packed by construction (8 chars + six u64)
  char magic[8];
  uint64_t in_total, out_total, weight_count, bias_count, vocab, embed_dim;
};
static_assert(sizeof(StockHeader) == 56, "stock header is 56 bytes");

struct MoeHeader {
  uint64_t magic, version, d_model, d_ff, num_experts, top_k, num_shared, flags, payload_bytes;
};

struct File {
  FILE* f = nullptr;
  ~File() {
    if (f) fclose(f);
  }
  bool open(const std::string& p, const char* mode) {
    f = fopen(p.c_str(), mode);
    return f != nullptr;
  }
  void close() {
    if (f) fclose(f);
    f = nullptr;
  }
};

bool mul_ok(uint64_t a, uint64_t b, uint64_t* out) {
  if (a != 0 && b > UINT64_MAX / a) return false;
  *out = a * b;
  return true;
}

int64_t file_size(FILE* f) {
  if (fseeko(f, 0, SEEK_END) != 0) return -1;
  const int64_t n = ftello(f);
  if (fseeko(f, 0, SEEK_SET) != 0) return -1;
  return n;
}

// Byte offset just past the stock payload (header, flat weights, bias, embeddings,
// transformer block).  Fails if the file is not a stock checkpoint with a
// transformer block, or is shorter than its own header says.
int stock_prefix_bytes(FILE* f, const char* path, int64_t total, int64_t* prefix) {
  StockHeader h;
  if (fread(&h, 1, sizeof(h), f) != sizeof(h)) return fail(AXM_ERR_ARGUMENT, "%s: shorter than the 56-byte header", path);
  if (memcmp(h.magic, "AXIOM_V1", 8) != 0) return fail(AXM_ERR_ARGUMENT, "%s: not an AXIOM_V1 checkpoint", path);
  uint64_t emb = 0, floats = 0;
  if (h.vocab > 0 && h.embed_dim > 0 && !mul_ok(h.vocab, h.embed_dim, &emb))
    return fail(AXM_ERR_ARGUMENT, "%s: embedding size overflows", path);
  floats = h.weight_count;
  if (floats + h.bias_count < floats) return fail(AXM_ERR_ARGUMENT, "%s: element counts overflow", path);
  floats += h.bias_count;
  if (floats + emb < floats) return fail(AXM_ERR_ARGUMENT, "%s: element counts overflow", path);
  floats += emb;
  if (floats > (uint64_t)total / 4) return fail(AXM_ERR_ARGUMENT, "%s: shorter than its header says", path);
  int64_t off = (int64_t)sizeof(h) + (int64_t)(floats * 4);
  if (off + 24 > total)
    return fail(AXM_ERR_ARGUMENT, "%s: no transformer block; the MoE block can only follow one", path);
  if (fseeko(f, off, SEEK_SET) != 0) return fail(AXM_ERR_ARGUMENT, "%s: seek failed", path);
  uint64_t tag[3];
  if (fread(tag, 8, 3, f) != 3 || tag[0] != kStockTag || tag[1] == 0 || tag[2] == 0)
    return fail(AXM_ERR_ARGUMENT, "%s: no valid transformer block after the embeddings", path);
  uint64_t dd, df, dd4, df3;
  if (!mul_ok(tag[1], tag[1], &dd) || !mul_ok(tag[1], tag[2], &df) || !mul_ok(dd, 4, &dd4) ||
      !mul_ok(df, 3, &df3) || dd4 + df3 < dd4 || dd4 + df3 > (uint64_t)total / 4)
    return fail(AXM_ERR_ARGUMENT, "%s: transformer block larger than the file", path);
  off += 24 + (int64_t)((dd4 + df3) * 4);
  if (off > total) return fail(AXM_ERR_ARGUMENT, "%s: transformer block is incomplete", path);
  *prefix = off;
  return AXM_OK;
}

struct Piece {
  const float* src;  // save
  float* dst;        // load
  uint64_t count;
  const char* name;
};

int check_shape(const AxmMoeDesc* d) {
  if (d == nullptr) return fail(AXM_ERR_ARGUMENT, "desc is null");
  if (d->d_model <= 0 || d->d_ff <= 0 || d->num_experts <= 0 || d->top_k <= 0 || d->num_shared < 0 ||
      d->top_k > d->num_experts)
    return fail(AXM_ERR_ARGUMENT, "checkpoint: bad layer shape (d_model %d, d_ff %d, experts %d, top_k %d, shared %d)",
                d->d_model, d->d_ff, d->num_experts, d->top_k, d->num_shared);
  return AXM_OK;
}

// The tensors of a block in file order.  `need_all`: every tensor the shape implies
// must have a buffer (the bias is optional: present in the file iff `with_bias`).
int list_pieces(const AxmMoeDesc* d, const AxmMoeCheckpoint* t, bool with_bias, std::vector<Piece>* out) {
  if (t == nullptr) return fail(AXM_ERR_ARGUMENT, "checkpoint: tensor table is null");
  const uint64_t D = d->d_model, F = d->d_ff, E = d->num_experts, S = d->num_shared;
  auto add = [&](float* p, uint64_t n, const char* name) -> int {
    if (p == nullptr) return fail(AXM_ERR_ARGUMENT, "checkpoint: %s is null", name);
    out->push_back(Piece{p, p, n, name});
    return AXM_OK;
  };
  int rc;
  if ((rc = add(t->router_w, D * E, "router_w"))) return rc;
  if (with_bias && (rc = add(t->router_bias, E, "router_bias"))) return rc;
  if ((rc = add(t->w_gate, E * D * F, "w_gate"))) return rc;
  if ((rc = add(t->w_up, E * D * F, "w_up"))) return rc;
  if ((rc = add(t->w_down, E * F * D, "w_down"))) return rc;
  if (S > 0) {
    if ((rc = add(t->shared_gate, S * D * F, "shared_gate"))) return rc;
    if ((rc = add(t->shared_up, S * D * F, "shared_up"))) return rc;
    if ((rc = add(t->shared_down, S * F * D, "shared_down"))) return rc;
  }
  return AXM_OK;
}

uint64_t payload_bytes_of(const AxmMoeDesc* d, bool with_bias) {
  const uint64_t D = d->d_model, F = d->d_ff, E = d->num_experts, S = d->num_shared;
  return 4 * (D * E + (with_bias ? E : 0) + 3 * E * D * F + 3 * S * D * F);
}

uint64_t word_sum(const float* p, size_t n) {
  uint64_t s = 0;
  const uint32_t* w = reinterpret_cast<const uint32_t*>(p);
  for (size_t i = 0; i < n; ++i) s += w[i];
  return s;
}

bool all_finite(const float* p, size_t n) {
  for (size_t i = 0; i < n; ++i)
    if (!std::isfinite(p[i])) return false;
  return true;
}

// Reads and validates the block header at `prefix`.  *found = false (and AXM_OK) when
// the file simply ends after the stock payload.
int read_moe_header(FILE* f, const char* path, int64_t prefix, int64_t total, MoeHeader* h, bool* found) {
  *found = false;
  if (prefix == total) return AXM_OK;
  if (fseeko(f, prefix, SEEK_SET) != 0) return fail(AXM_ERR_ARGUMENT, "%s: seek failed", path);
  if (total - prefix < (int64_t)sizeof(MoeHeader) || fread(h, 1, sizeof(*h), f) != sizeof(*h))
    return fail(AXM_ERR_ARGUMENT, "%s: trailing bytes after the transformer block are not an MoE block", path);
  if (h->magic != kMoeTag) return fail(AXM_ERR_ARGUMENT, "%s: unknown tag after the transformer block", path);
  if (h->version != kMoeVersion)
    return fail(AXM_ERR_ARGUMENT, "%s: MoE block version %llu, this library reads %llu", path,
                (unsigned long long)h->version, (unsigned long long)kMoeVersion);
  const uint64_t lim = 1u << 30;
  if (h->d_model == 0 || h->d_ff == 0 || h->num_experts == 0 || h->top_k == 0 || h->d_model > lim ||
      h->d_ff > lim || h->num_experts > lim || h->top_k > h->num_experts || h->num_shared > lim || (h->flags & ~1ULL))
    return fail(AXM_ERR_ARGUMENT, "%s: MoE block header holds impossible sizes", path);
  AxmMoeDesc d{};
  d.d_model = (int32_t)h->d_model;
  d.d_ff = (int32_t)h->d_ff;
  d.num_experts = (int32_t)h->num_experts;
  d.top_k = (int32_t)h->top_k;
  d.num_shared = (int32_t)h->num_shared;
  // 3 * (E + S) * D * F elements must fit in the file, which also rules out overflow
  uint64_t df, edf;
  if (!mul_ok(h->d_model, h->d_ff, &df) || !mul_ok(df, 3 * (h->num_experts + h->num_shared), &edf) ||
      edf > (uint64_t)total / 4)
    return fail(AXM_ERR_ARGUMENT, "%s: MoE block larger than the file", path);
  if (h->payload_bytes != payload_bytes_of(&d, (h->flags & 1) != 0))
    return fail(AXM_ERR_ARGUMENT, "%s: MoE block payload size does not match its shape", path);
  if ((uint64_t)(total - prefix) != sizeof(MoeHeader) + h->payload_bytes + 8)
    return fail(AXM_ERR_ARGUMENT, "%s: MoE block is incomplete or followed by unknown bytes", path);
  *found = true;
  return AXM_OK;
}

__global__ void cast_master_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = __float2bfloat16_rn(src[i]);
}

}  // namespace
}  // namespace axm

using namespace axm;

extern "C" int axm_moe_checkpoint_save(const char* path, const AxmMoeDesc* desc,
                                       const AxmMoeCheckpoint* tensors) {
  if (path == nullptr || path[0] == 0) return fail(AXM_ERR_ARGUMENT, "checkpoint: path is empty");
  if (int rc = check_shape(desc)) return rc;
  const bool with_bias = tensors != nullptr && tensors->router_bias != nullptr;
  std::vector<Piece> pieces;
  if (int rc = list_pieces(desc, tensors, with_bias, &pieces)) return rc;
  // refuse to write a damaged checkpoint (as the engine's writer does for its own tensors)
  for (const Piece& p : pieces)
    if (!all_finite(p.src, p.count))
      return fail(AXM_ERR_ARGUMENT, "checkpoint: %s contains NaN or Inf; nothing written", p.name);

  File in;
  if (!in.open(path, "rb")) return fail(AXM_ERR_ARGUMENT, "%s: cannot open (%s)", path, strerror(errno));
  const int64_t total = file_size(in.f);
  if (total < 0) return fail(AXM_ERR_ARGUMENT, "%s: cannot determine the size", path);
  int64_t prefix = 0;
  if (int rc = stock_prefix_bytes(in.f, path, total, &prefix)) return rc;
  MoeHeader old;
  bool found = false;
  if (int rc = read_moe_header(in.f, path, prefix, total, &old, &found)) return rc;  // damaged tail: do not guess

  const std::string tmp = std::string(path) + ".tmp";
  File out;
  if (!out.open(tmp, "wb")) return fail(AXM_ERR_ARGUMENT, "%s: cannot open for writing (%s)", tmp.c_str(), strerror(errno));
  auto abandon = [&](const char* what) {
    out.close();
    remove(tmp.c_str());
    return fail(AXM_ERR_ARGUMENT, "%s: %s; %s left untouched", tmp.c_str(), what, path);
  };
  // 1. the stock payload, byte for byte
  if (fseeko(in.f, 0, SEEK_SET) != 0) return abandon("seek failed");
  std::vector<char> buf(4u << 20);
  for (int64_t left = prefix; left > 0;) {
    const size_t n = (size_t)(left < (int64_t)buf.size() ? left : (int64_t)buf.size());
    if (fread(buf.data(), 1, n, in.f) != n) return abandon("short read of the existing checkpoint");
    if (fwrite(buf.data(), 1, n, out.f) != n) return abandon("write failed");
    left -= (int64_t)n;
  }
  // 2. the MoE block
  MoeHeader h;
  h.magic = kMoeTag;
  h.version = kMoeVersion;
  h.d_model = (uint64_t)desc->d_model;
  h.d_ff = (uint64_t)desc->d_ff;
  h.num_experts = (uint64_t)desc->num_experts;
  h.top_k = (uint64_t)desc->top_k;
  h.num_shared = (uint64_t)desc->num_shared;
  h.flags = with_bias ? 1 : 0;
  h.payload_bytes = payload_bytes_of(desc, with_bias);
  if (fwrite(&h, 1, sizeof(h), out.f) != sizeof(h)) return abandon("write failed");
  uint64_t sum = 0;
  for (const Piece& p : pieces) {
    for (uint64_t done = 0; done < p.count; done += kChunkFloats) {
      const size_t n = (size_t)(p.count - done < kChunkFloats ? p.count - done : kChunkFloats);
      if (fwrite(p.src + done, 4, n, out.f) != n) return abandon("write failed");
      sum += word_sum(p.src + done, n);
    }
  }
  if (fwrite(&sum, 1, 8, out.f) != 8) return abandon("write failed");
  if (fflush(out.f) != 0) return abandon("flush failed");
  out.close();
  in.close();
  // 3. replace the target
  if (rename(tmp.c_str(), path) != 0) {
    const int e = errno;
    remove(tmp.c_str());
    return fail(AXM_ERR_ARGUMENT, "%s: rename over %s failed (%s)", tmp.c_str(), path, strerror(e));
  }
  return AXM_OK;
}

extern "C" int axm_moe_checkpoint_probe(const char* path, AxmMoeDesc* desc, int32_t* has_bias) {
  if (path == nullptr || desc == nullptr) return fail(AXM_ERR_ARGUMENT, "checkpoint: null argument");
  File in;
  if (!in.open(path, "rb")) return fail(AXM_ERR_ARGUMENT, "%s: cannot open (%s)", path, strerror(errno));
  const int64_t total = file_size(in.f);
  if (total < 0) return fail(AXM_ERR_ARGUMENT, "%s: cannot determine the size", path);
  int64_t prefix = 0;
  if (int rc = stock_prefix_bytes(in.f, path, total, &prefix)) return rc;
  MoeHeader h;
  bool found = false;
  if (int rc = read_moe_header(in.f, path, prefix, total, &h, &found)) return rc;
  if (!found) return fail(AXM_ERR_ARGUMENT, "%s: holds no MoE block", path);
  desc->d_model = (int32_t)h.d_model;
  desc->d_ff = (int32_t)h.d_ff;
  desc->num_experts = (int32_t)h.num_experts;
  desc->top_k = (int32_t)h.top_k;
  desc->num_shared = (int32_t)h.num_shared;
  if (has_bias != nullptr) *has_bias = (int32_t)(h.flags & 1);
  return AXM_OK;
}

extern "C" int axm_moe_checkpoint_load(const char* path, const AxmMoeDesc* desc,
                                       const AxmMoeCheckpoint* tensors) {
  if (path == nullptr) return fail(AXM_ERR_ARGUMENT, "checkpoint: path is null");
  if (int rc = check_shape(desc)) return rc;
  File in;
  if (!in.open(path, "rb")) return fail(AXM_ERR_ARGUMENT, "%s: cannot open (%s)", path, strerror(errno));
  const int64_t total = file_size(in.f);
  if (total < 0) return fail(AXM_ERR_ARGUMENT, "%s: cannot determine the size", path);
  int64_t prefix = 0;
  if (int rc = stock_prefix_bytes(in.f, path, total, &prefix)) return rc;
  MoeHeader h;
  bool found = false;
  if (int rc = read_moe_header(in.f, path, prefix, total, &h, &found)) return rc;
  if (!found) return fail(AXM_ERR_ARGUMENT, "%s: holds no MoE block", path);
  if (h.d_model != (uint64_t)desc->d_model || h.d_ff != (uint64_t)desc->d_ff ||
      h.num_experts != (uint64_t)desc->num_experts || h.top_k != (uint64_t)desc->top_k ||
      h.num_shared != (uint64_t)desc->num_shared)
    return fail(AXM_ERR_ARGUMENT,
                "%s: MoE block is d_model %llu, d_ff %llu, %llu experts, top-%llu, %llu shared; the layer is %d, %d, %d, top-%d, %d",
                path, (unsigned long long)h.d_model, (unsigned long long)h.d_ff, (unsigned long long)h.num_experts,
                (unsigned long long)h.top_k, (unsigned long long)h.num_shared, desc->d_model, desc->d_ff,
                desc->num_experts, desc->top_k, desc->num_shared);
  const bool with_bias = (h.flags & 1) != 0;
  std::vector<Piece> pieces;
  if (int rc = list_pieces(desc, tensors, with_bias, &pieces)) return rc;
  uint64_t sum = 0;
  bool finite = true;
  for (const Piece& p : pieces) {
    for (uint64_t done = 0; done < p.count; done += kChunkFloats) {
      const size_t n = (size_t)(p.count - done < kChunkFloats ? p.count - done : kChunkFloats);
      if (fread(p.dst + done, 4, n, in.f) != n) return fail(AXM_ERR_ARGUMENT, "%s: short read in %s", path, p.name);
      sum += word_sum(p.dst + done, n);
      finite = finite && all_finite(p.dst + done, n);
    }
  }
  uint64_t stored = 0;
  if (fread(&stored, 1, 8, in.f) != 8) return fail(AXM_ERR_ARGUMENT, "%s: checksum missing", path);
  if (stored != sum) return fail(AXM_ERR_ARGUMENT, "%s: MoE block checksum mismatch; the buffers hold damaged data", path);
  if (!finite) return fail(AXM_ERR_ARGUMENT, "%s: MoE block contains NaN or Inf; the buffers hold damaged data", path);
  return AXM_OK;
}

extern "C" int axm_moe_cast_master(const float* master, void* w_bf16, size_t n, void* stream) {
  if (master == nullptr || w_bf16 == nullptr) return fail(AXM_ERR_ARGUMENT, "axm_moe_cast_master: null pointer");
  if (n == 0) return AXM_OK;
  if (int rc = require_device()) return rc;
  size_t blocks = (n + 1023) / 1024;
  const size_t cap = (size_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  cast_master_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      master, static_cast<__nv_bfloat16*>(w_bf16), n);
  return check_launch("cast_master_kernel");
}
