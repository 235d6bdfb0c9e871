// Minimal reader of the safetensors container (8-byte little-endian header length, JSON header mapping
// tensor name -> {dtype, shape, data_offsets}, raw little-endian data) and the model loader built on
// it. Counterpart of the reference's flux_safetensors.c:155-292 + flux_transformer_load_safetensors
// (flux_transformer.c:4411-4656), except that tensors go to the GPU as bf16 instead of being
// expanded to f32 in host memory, and that every shape is validated.
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <functional>
#include <string>
#include <vector>

#include "engine.cuh"
#include "flux_cuda.h"

namespace fx {

struct StEntry {
  std::string name, dtype;
  std::vector<long long> shape;
  unsigned long long begin = 0, end = 0;
};

// Recursive-descent parser for the subset of JSON a safetensors header uses.
struct JsonCursor {
  const char *p, *e;
  bool ok = true;
  void ws() {
    while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  bool eat(char c) {
    ws();
    if (p < e && *p == c) {
      ++p;
      return true;
    }
    return false;
  }
  std::string str() {
    ws();
    std::string s;
    if (p >= e || *p != '"') {
      ok = false;
      return s;
    }
    ++p;
    while (p < e && *p != '"') {
      if (*p == '\\' && p + 1 < e) {
        ++p;
        switch (*p) {
          case 'n': s += '\n'; break;
          case 't': s += '\t'; break;
          case 'u': p += (p + 4 < e) ? 4 : 0; s += '?'; break;
          default: s += *p;
        }
        ++p;
      } else {
        s += *p++;
      }
    }
    if (p >= e) ok = false;
    else ++p;
    return s;
  }
  long long num() {
    ws();
    long long v = 0;
    bool any = false;
    while (p < e && *p >= '0' && *p <= '9') {
      v = v * 10 + (*p++ - '0');
      any = true;
    }
    if (!any) ok = false;
    return v;
  }
  void skip_value() {  // used for __metadata__
    ws();
    if (p >= e) {
      ok = false;
      return;
    }
    if (*p == '"') {
      str();
    } else if (*p == '{' || *p == '[') {
      const char open = *p, close = (*p == '{') ? '}' : ']';
      int depth = 0;
      bool in_str = false;
      for (; p < e; ++p) {
        if (in_str) {
          if (*p == '\\') ++p;
          else if (*p == '"') in_str = false;
        } else if (*p == '"') in_str = true;
        else if (*p == open) ++depth;
        else if (*p == close && --depth == 0) {
          ++p;
          return;
        }
      }
      ok = false;
    } else {
      while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;
    }
  }
};

static bool parse_header(const char *js, size_t len, std::vector<StEntry> &out) {
  JsonCursor c{js, js + len};
  if (!c.eat('{')) return false;
  if (c.eat('}')) return true;
  do {
    StEntry en;
    en.name = c.str();
    if (!c.ok || !c.eat(':')) return false;
    if (en.name == "__metadata__") {
      c.skip_value();
      if (!c.ok) return false;
      continue;
    }
    if (!c.eat('{')) return false;
    do {
      std::string key = c.str();
      if (!c.ok || !c.eat(':')) return false;
      if (key == "dtype") {
        en.dtype = c.str();
      } else if (key == "shape") {
        if (!c.eat('[')) return false;
        if (!c.eat(']')) {
          do en.shape.push_back(c.num());
          while (c.eat(','));
          if (!c.eat(']')) return false;
        }
      } else if (key == "data_offsets") {
        if (!c.eat('[')) return false;
        en.begin = static_cast<unsigned long long>(c.num());
        if (!c.eat(',')) return false;
        en.end = static_cast<unsigned long long>(c.num());
        if (!c.eat(']')) return false;
      } else {
        c.skip_value();
      }
      if (!c.ok) return false;
    } while (c.eat(','));
    if (!c.eat('}')) return false;
    out.push_back(en);
  } while (c.eat(','));
  return c.eat('}') && c.ok;
}

static int infer_dims(const std::vector<StEntry> &es, ModelDims &d) {
  memset(&d, 0, sizeof(d));
  d.head_dim = 128;
  d.rope_theta = 2000.0f;
  d.axis_dim = 32;
  for (const StEntry &e : es) {
    int idx;
    if (e.name == "x_embedder.weight" && e.shape.size() == 2) {
      d.hidden = static_cast<int>(e.shape[0]);
      d.latent_ch = static_cast<int>(e.shape[1]);
    } else if (e.name == "context_embedder.weight" && e.shape.size() == 2) {
      d.text_dim = static_cast<int>(e.shape[1]);
    } else if (e.name == "time_guidance_embed.timestep_embedder.linear_1.weight" && e.shape.size() == 2) {
      d.time_dim = static_cast<int>(e.shape[1]);
    } else if (e.name == "transformer_blocks.0.ff.linear_out.weight" && e.shape.size() == 2) {
      d.mlp = static_cast<int>(e.shape[1]);
    } else if (e.name == "single_transformer_blocks.0.attn.to_out.weight" && e.shape.size() == 2 && !d.mlp) {
      d.mlp = static_cast<int>(e.shape[1] - e.shape[0]);
    }
    if (sscanf(e.name.c_str(), "transformer_blocks.%d.", &idx) == 1 && idx + 1 > d.n_double) d.n_double = idx + 1;
    if (sscanf(e.name.c_str(), "single_transformer_blocks.%d.", &idx) == 1 && idx + 1 > d.n_single)
      d.n_single = idx + 1;
  }
  if (!d.hidden || !d.latent_ch || !d.text_dim || !d.time_dim || !d.mlp) return -1;
  d.heads = d.hidden / d.head_dim;
  return 0;
}

// Maps `path`, parses its header and calls visit(name, data, dtype 0/1/2 = F32/F16/BF16, shape, ndim) for every
// tensor; stops at the first non-zero return. Tensors of other dtypes or ranks are reported as errors.
int safetensors_for_each(const char *path,
                         const std::function<int(const char *, const void *, int, const long long *, int)> &visit) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) {
    set_error("cannot open %s", path);
    return FLUX_CUDA_ERR_IO;
  }
  struct stat sb;
  if (fstat(fd, &sb) != 0 || sb.st_size < 10) {
    close(fd);
    set_error("%s: too short to be a safetensors file", path);
    return FLUX_CUDA_ERR_IO;
  }
  const size_t fsize = static_cast<size_t>(sb.st_size);
  void *map = mmap(nullptr, fsize, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (map == MAP_FAILED) {
    set_error("%s: mmap failed", path);
    return FLUX_CUDA_ERR_IO;
  }
  const unsigned char *base = reinterpret_cast<const unsigned char *>(map);
  unsigned long long hlen = 0;
  for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | base[i];
  int rc = 0;
  std::vector<StEntry> es;
  if (hlen == 0 || hlen > fsize - 8 || hlen > (100ull << 20)) {
    set_error("%s: implausible header length %llu", path, hlen);
    rc = FLUX_CUDA_ERR_IO;
  } else if (!parse_header(reinterpret_cast<const char *>(base + 8), hlen, es)) {
    set_error("%s: malformed header", path);
    rc = FLUX_CUDA_ERR_IO;
  }
  const size_t data0 = 8 + hlen;
  for (size_t i = 0; !rc && i < es.size(); ++i) {
    const StEntry &e = es[i];
    const int dt = e.dtype == "F32" ? 0 : e.dtype == "F16" ? 1 : e.dtype == "BF16" ? 2 : -1;
    size_t count = 1;
    for (long long d : e.shape) count *= static_cast<size_t>(d);
    const size_t esz = dt == 0 ? 4 : 2;
    if (dt < 0 || e.shape.empty() || e.shape.size() > 4) {  // the visitor judges the rank it expects
      set_error("%s: tensor %s has unsupported dtype/rank", path, e.name.c_str());
      rc = FLUX_CUDA_ERR_MODEL;
    } else if (e.end < e.begin || e.end - e.begin != count * esz || data0 + e.end > fsize) {
      set_error("%s: tensor %s has inconsistent offsets (file truncated?)", path, e.name.c_str());
      rc = FLUX_CUDA_ERR_IO;
    } else {
      rc = visit(e.name.c_str(), base + data0 + e.begin, dt, e.shape.data(), static_cast<int>(e.shape.size()));
    }
  }
  munmap(map, fsize);
  return rc;
}

int model_load_safetensors(flux_cuda_ctx *ctx, const char *path, flux_cuda_model **out) {
  *out = nullptr;
  if (!ctx || !path) return FLUX_CUDA_ERR_ARG;
  int fd = open(path, O_RDONLY);
  if (fd < 0) {
    set_error("cannot open %s", path);
    return FLUX_CUDA_ERR_IO;
  }
  struct stat sb;
  if (fstat(fd, &sb) != 0 || sb.st_size < 10) {
    close(fd);
    set_error("%s: too short to be a safetensors file", path);
    return FLUX_CUDA_ERR_IO;
  }
  const size_t fsize = static_cast<size_t>(sb.st_size);
  void *map = mmap(nullptr, fsize, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (map == MAP_FAILED) {
    set_error("%s: mmap failed", path);
    return FLUX_CUDA_ERR_IO;
  }
  const unsigned char *base = reinterpret_cast<const unsigned char *>(map);
  unsigned long long hlen = 0;
  for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | base[i];
  int rc = 0;
  flux_cuda_model *m = nullptr;
  std::vector<StEntry> es;
  if (hlen == 0 || hlen > fsize - 8 || hlen > (100ull << 20)) {
    set_error("%s: implausible header length %llu", path, hlen);
    rc = FLUX_CUDA_ERR_IO;
  } else if (!parse_header(reinterpret_cast<const char *>(base + 8), hlen, es)) {
    set_error("%s: malformed header", path);
    rc = FLUX_CUDA_ERR_IO;
  }
  ModelDims d;
  if (!rc && infer_dims(es, d)) {
    set_error("%s: cannot infer model dimensions (embedder / block tensors missing)", path);
    rc = FLUX_CUDA_ERR_MODEL;
  }
  if (!rc) rc = model_create(ctx, d, &m);
  const size_t data0 = 8 + hlen;
  for (size_t i = 0; !rc && i < es.size(); ++i) {
    const StEntry &e = es[i];
    int dt = e.dtype == "F32" ? 0 : e.dtype == "F16" ? 1 : e.dtype == "BF16" ? 2 : -1;
    size_t count = 1;
    for (long long s : e.shape) count *= static_cast<size_t>(s);
    const size_t esz = dt == 0 ? 4 : 2;
    if (dt < 0 || e.shape.empty() || e.shape.size() > 2) {
      set_error("%s: tensor %s has unsupported dtype/rank", path, e.name.c_str());
      rc = FLUX_CUDA_ERR_MODEL;
    } else if (e.end < e.begin || e.end - e.begin != count * esz || data0 + e.end > fsize) {
      set_error("%s: tensor %s has inconsistent offsets (file truncated?)", path, e.name.c_str());
      rc = FLUX_CUDA_ERR_IO;
    } else {
      rc = model_set_tensor(m, e.name.c_str(), base + data0 + e.begin, dt, e.shape.data(),
                            static_cast<int>(e.shape.size()));
    }
  }
  if (!rc) rc = model_finalize(m);
  munmap(map, fsize);
  if (rc) {
    model_free(m);
    return rc;
  }
  *out = m;
  return 0;
}

}  // namespace fx
