// Several GPUs of one machine behind the C ABI: independent images on replicas, and the guidance pair of the base
// model split across two GPUs.
//
// The reference is single-device: its guided sampler runs the unconditional and the conditional pass one after the
// other (flux_sample_euler_cfg, flux_sample.c:457-529), and a batch of images is a host loop. Here one host thread
// drives each GPU through its own context. Independent images need no exchange at all. The guidance pair exchanges
// ONE velocity per step: each GPU scales its velocity (g on the conditional side, 1 - g on the other), stores it
// straight into the other GPU's memory over NVLink with plain stores, raises a flag there, waits for the flag the
// other side raises here, and adds the two halves into its own copy of the latent - one kernel per step and GPU
// (pair_exchange_euler_kernel). a + b is computed from the same two operands on both sides, so the two latents stay
// bit-identical without ever being compared.
//
// Liveness. Before a GPU is given the kernel that waits for its peer, the two host threads meet in a rendezvous with
// a time limit (flux_cuda_rendezvous_*): a thread whose partner failed, or never arrives, returns
// FLUX_CUDA_ERR_PEER_TIMEOUT without having launched anything that waits. The wait inside the kernel is bounded as
// well (~2 s of SM clock); when it runs out the kernel records KERR_PEER_TIMEOUT, skips the update and returns.
// Only plain loads and stores touch the peer's memory: no TMA, no multicast.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <condition_variable>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "context.cuh"
#include "engine.cuh"
#include "flux_cuda.h"
#include "ptx.cuh"

// ------------------------------------------------------------------------------------------------ rendezvous
struct flux_cuda_rendezvous {
  std::mutex m;
  std::condition_variable cv;
  std::vector<long long> at;  // last sequence number each party announced
  std::vector<char> gone;     // party gave up (its work failed): nobody should wait for it again
};

extern "C" {

int flux_cuda_rendezvous_create(int parties, flux_cuda_rendezvous **out) {
  if (!out || parties < 1 || parties > 64) {
    fx::set_error("rendezvous: 1 to 64 parties");
    return FLUX_CUDA_ERR_ARG;
  }
  flux_cuda_rendezvous *r = new flux_cuda_rendezvous();
  r->at.assign(parties, -1);
  r->gone.assign(parties, 0);
  *out = r;
  return FLUX_CUDA_OK;
}

void flux_cuda_rendezvous_destroy(flux_cuda_rendezvous *r) { delete r; }

int flux_cuda_rendezvous_arrive_and_wait(flux_cuda_rendezvous *r, int party, long long seq, int timeout_ms) {
  if (!r || party < 0 || party >= static_cast<int>(r->at.size()) || timeout_ms < 0) {
    fx::set_error("rendezvous: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  std::unique_lock<std::mutex> lk(r->m);
  r->at[party] = seq;
  r->cv.notify_all();
  int missing = -1, left = -1;
  auto settled = [&]() {
    missing = left = -1;
    for (int o = 0; o < static_cast<int>(r->at.size()); ++o) {
      if (o == party || r->at[o] >= seq) continue;
      if (r->gone[o]) left = o;
      else missing = o;
    }
    return left >= 0 || missing < 0;
  };
  const bool in_time = r->cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), settled);
  if (left >= 0) {
    fx::set_error("peer %d gave up before step %lld: nothing that waits for it was launched", left, seq);
    return FLUX_CUDA_ERR_PEER_TIMEOUT;
  }
  if (!in_time) {
    fx::set_error("peer %d did not reach step %lld within %d ms: nothing that waits for it was launched", missing, seq,
                  timeout_ms);
    return FLUX_CUDA_ERR_PEER_TIMEOUT;
  }
  return FLUX_CUDA_OK;
}

void flux_cuda_rendezvous_abandon(flux_cuda_rendezvous *r, int party) {
  if (!r || party < 0 || party >= static_cast<int>(r->at.size())) return;
  std::lock_guard<std::mutex> lk(r->m);
  r->gone[party] = 1;
  r->cv.notify_all();
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------ device side
namespace fx {

// One step of one member of a guidance pair, after its forward pass.
//   own = coef * v;  peer_inbox[i] = own (plain stores into the other GPU's memory);  peer_flag = seq once every
//   block's stores are out;  wait (bounded) until my_flag >= seq;  z += dt * (own + my_inbox).
// All blocks are co-resident (the grid is far smaller than the device) and the peer runs the same kernel on its own
// GPU, so the wait ends as soon as the peer's stores have landed.
__global__ void __launch_bounds__(256) pair_exchange_euler_kernel(float *__restrict__ z, const float *__restrict__ v,
                                                                  float coef, const float *__restrict__ sched, int step,
                                                                  long long n, float *peer_inbox, int *peer_flag,
                                                                  const float *my_inbox, const int *my_flag,
                                                                  unsigned int *block_counter, int seq, int *err,
                                                                  long long limit_cycles) {
  __shared__ int s_ok;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  // __fmul_rn / __fadd_rn: never contracted into a fused multiply-add, so that both GPUs add the very same two
  // rounded halves and their latents stay bit-identical
  for (long long i = i0; i < n; i += stride) peer_inbox[i] = __fmul_rn(coef, v[i]);
  __threadfence_system();  // this thread's stores are visible system-wide before the block counts itself
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int arrived = atomicAdd(block_counter, 1u);
    if (arrived == gridDim.x - 1) {  // last block: every block's stores are out
      *block_counter = 0;            // ready for the next launch on this stream
      __threadfence_system();
      *reinterpret_cast<volatile int *>(peer_flag) = seq;
    }
    const volatile int *flag = my_flag;
    int ok = 1;
    if (*flag < seq) {
      const long long t0 = clock64();
      while (*flag < seq) {
        if (clock64() - t0 > limit_cycles) {
          ok = 0;
          break;
        }
        __nanosleep(200);
      }
    }
    if (!ok) atomicCAS(err, 0, KERR_PEER_TIMEOUT);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;  // the peer's half never arrived: leave the latent as it is
  __threadfence_system();
  const float dt = sched[step + 1] - sched[step];
  for (long long i = i0; i < n; i += stride) {
    const float own = __fmul_rn(coef, v[i]);
    const float other = __ldcv(my_inbox + i);
    z[i] = fmaf(dt, __fadd_rn(own, other), z[i]);
  }
}

}  // namespace fx

// ------------------------------------------------------------------------------------------------ group
struct flux_cuda_group {
  std::vector<flux_cuda_ctx *> ctx;
  std::vector<flux_cuda_model *> model;
  bool owns_models = false;
  // guidance pair (members 0 and 1): per member an inbox of two slots (step parity), a flag and a block counter,
  // all in that member's own memory; the peer reaches inbox and flag through peer access
  float *inbox[2] = {nullptr, nullptr};
  int *flag[2] = {nullptr, nullptr};
  unsigned int *counter[2] = {nullptr, nullptr};
  size_t inbox_floats = 0;  // per slot
  bool peer_ok = false;
  int seq = 0;  // steps exchanged so far; flags only ever grow, so nothing has to be reset between images
  flux_cuda_rendezvous *rv = nullptr;
  int timeout_ms = 20000;
};

namespace {

using namespace fx;

struct WorkerResult {
  int rc = 0;
  std::string msg;
};

void note(WorkerResult &r, int rc) {
  if (rc && !r.rc) {
    r.rc = rc;
    r.msg = flux_cuda_last_error();
  }
}

// Starts a host thread; a failure to create one becomes an error of that member instead of an exception (nothing may
// throw through the C ABI).
template <class F>
bool spawn(std::thread &t, WorkerResult &r, F &&f) {
  try {
    t = std::thread(std::forward<F>(f));
    return true;
  } catch (...) {
    if (!r.rc) {
      r.rc = FLUX_CUDA_ERR_NOMEM;
      r.msg = "could not start a host thread for this GPU";
    }
    return false;
  }
}

int pair_buffers(flux_cuda_group *g, size_t floats) {
  if (g->inbox_floats >= floats) return 0;
  for (int r = 0; r < 2; ++r) {
    cudaSetDevice(g->ctx[r]->device);
    cudaStreamSynchronize(g->ctx[r]->stream);
    if (g->inbox[r]) cudaFree(g->inbox[r]);
    g->inbox[r] = nullptr;
    int rc = check_cuda(cudaMalloc(&g->inbox[r], 2 * floats * sizeof(float)), "cudaMalloc (pair inbox)");
    if (!rc && !g->flag[r]) {
      rc = check_cuda(cudaMalloc(&g->flag[r], sizeof(int)), "cudaMalloc (pair flag)");
      if (!rc) rc = check_cuda(cudaMalloc(&g->counter[r], sizeof(unsigned int)), "cudaMalloc (pair counter)");
      if (!rc) rc = check_cuda(cudaMemset(g->flag[r], 0, sizeof(int)), "cudaMemset");
      if (!rc) rc = check_cuda(cudaMemset(g->counter[r], 0, sizeof(unsigned int)), "cudaMemset");
      if (!rc) rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    }
    if (rc) return rc;
  }
  g->inbox_floats = floats;
  return 0;
}

}  // namespace

extern "C" {

int flux_cuda_group_create(int n_gpus, const int *devices, flux_cuda_group **out) {
  if (!out || n_gpus < 1 || n_gpus > 64) {
    set_error("group: 1 to 64 GPUs");
    return FLUX_CUDA_ERR_ARG;
  }
  *out = nullptr;
  flux_cuda_group *g = new flux_cuda_group();
  int rc = 0;
  for (int i = 0; i < n_gpus && !rc; ++i) {
    for (int j = 0; j < i && devices; ++j)
      if (devices[j] == devices[i]) {
        set_error("group: device %d is listed twice", devices[i]);
        rc = FLUX_CUDA_ERR_ARG;
      }
    flux_cuda_ctx *c = nullptr;
    if (!rc) rc = flux_cuda_ctx_create(devices ? devices[i] : i, &c);
    if (!rc) g->ctx.push_back(c);
  }
  if (!rc) rc = flux_cuda_rendezvous_create(2, &g->rv);
  if (!rc && n_gpus >= 2) {
    // the pair exchanges through peer memory: members 0 and 1 must reach each other
    const int d0 = g->ctx[0]->device, d1 = g->ctx[1]->device;
    int a01 = 0, a10 = 0;
    cudaDeviceCanAccessPeer(&a01, d0, d1);
    cudaDeviceCanAccessPeer(&a10, d1, d0);
    if (a01 && a10) {
      cudaSetDevice(d0);
      cudaError_t e0 = cudaDeviceEnablePeerAccess(d1, 0);
      cudaSetDevice(d1);
      cudaError_t e1 = cudaDeviceEnablePeerAccess(d0, 0);
      cudaGetLastError();  // "already enabled" is fine
      g->peer_ok = (e0 == cudaSuccess || e0 == cudaErrorPeerAccessAlreadyEnabled) &&
                   (e1 == cudaSuccess || e1 == cudaErrorPeerAccessAlreadyEnabled);
    }
  }
  if (const char *e = getenv("FLUX_CUDA_PEER_TIMEOUT_MS")) g->timeout_ms = atoi(e) > 0 ? atoi(e) : g->timeout_ms;
  if (rc) {
    flux_cuda_group_destroy(g);
    return rc;
  }
  g->model.assign(g->ctx.size(), nullptr);
  *out = g;
  return FLUX_CUDA_OK;
}

void flux_cuda_group_destroy(flux_cuda_group *g) {
  if (!g) return;
  for (size_t i = 0; i < g->model.size(); ++i)
    if (g->owns_models && g->model[i]) flux_cuda_model_free(g->model[i]);
  for (int r = 0; r < 2 && r < static_cast<int>(g->ctx.size()); ++r) {
    cudaSetDevice(g->ctx[r]->device);
    cudaStreamSynchronize(g->ctx[r]->stream);
    if (g->inbox[r]) cudaFree(g->inbox[r]);
    if (g->flag[r]) cudaFree(g->flag[r]);
    if (g->counter[r]) cudaFree(g->counter[r]);
  }
  for (flux_cuda_ctx *c : g->ctx) flux_cuda_ctx_destroy(c);
  flux_cuda_rendezvous_destroy(g->rv);
  delete g;
}

int flux_cuda_group_size(const flux_cuda_group *g) { return g ? static_cast<int>(g->ctx.size()) : 0; }

flux_cuda_ctx *flux_cuda_group_context(flux_cuda_group *g, int member) {
  return (g && member >= 0 && member < static_cast<int>(g->ctx.size())) ? g->ctx[member] : nullptr;
}

int flux_cuda_group_load_safetensors(flux_cuda_group *g, const char *path) {
  if (!g || !path) return FLUX_CUDA_ERR_ARG;
  const int n = static_cast<int>(g->ctx.size());
  std::vector<WorkerResult> res(n);
  std::vector<flux_cuda_model *> loaded(n, nullptr);
  std::vector<std::thread> th(n);
  for (int r = 0; r < n; ++r)
    spawn(th[r], res[r], [&, r]() { note(res[r], flux_cuda_model_load_safetensors(g->ctx[r], path, &loaded[r])); });
  for (auto &t : th)
    if (t.joinable()) t.join();
  for (int r = 0; r < n; ++r)
    if (res[r].rc) {
      for (flux_cuda_model *m : loaded) flux_cuda_model_free(m);
      set_error("GPU member %d: %s", r, res[r].msg.c_str());
      return res[r].rc;
    }
  for (int r = 0; r < n; ++r) {
    if (g->owns_models && g->model[r]) flux_cuda_model_free(g->model[r]);
    g->model[r] = loaded[r];
  }
  g->owns_models = true;
  return FLUX_CUDA_OK;
}

flux_cuda_model *flux_cuda_group_model(flux_cuda_group *g, int member) {
  return (g && member >= 0 && member < static_cast<int>(g->model.size())) ? g->model[member] : nullptr;
}

void flux_cuda_group_unload(flux_cuda_group *g) {
  if (!g) return;
  for (size_t r = 0; r < g->model.size(); ++r) {
    if (g->owns_models && g->model[r]) flux_cuda_model_free(g->model[r]);
    g->model[r] = nullptr;
  }
  g->owns_models = false;
}

int flux_cuda_group_set_models(flux_cuda_group *g, flux_cuda_model *const *models) {
  if (!g || !models) return FLUX_CUDA_ERR_ARG;
  for (size_t r = 0; r < g->ctx.size(); ++r) {
    if (!models[r] || models[r]->ctx != g->ctx[r]) {
      set_error("group: model %zu was not created from the group's context %zu", r, r);
      return FLUX_CUDA_ERR_ARG;
    }
  }
  for (size_t r = 0; r < g->ctx.size(); ++r) {
    if (g->owns_models && g->model[r]) flux_cuda_model_free(g->model[r]);
    g->model[r] = models[r];
  }
  g->owns_models = false;
  return FLUX_CUDA_OK;
}

int flux_cuda_group_sample_batch(flux_cuda_group *g, const flux_cuda_sample_params *p, int n_images,
                                 const float *const *z0, const float *const *ctx, float *const *latent_out) {
  if (!g || !p || n_images < 0 || (n_images && (!z0 || !ctx || !latent_out)) || !p->schedule || p->ctx_uncond) {
    set_error("group_sample_batch: bad argument (guided sampling goes through flux_cuda_group_sample_cfg_pair)");
    return FLUX_CUDA_ERR_ARG;
  }
  const int n = static_cast<int>(g->ctx.size());
  for (int r = 0; r < n; ++r)
    if (!g->model[r]) {
      set_error("group: no model on member %d", r);
      return FLUX_CUDA_ERR_MODEL;
    }
  std::vector<WorkerResult> res(n);
  std::vector<std::thread> th(n);
  for (int r = 0; r < n && r < n_images; ++r)
    spawn(th[r], res[r], [&, r]() {
      // image i runs on member i % n; each member keeps one sampler for the whole batch
      std::vector<flux_cuda_ref_shape> shapes;
      std::vector<const float *> lat;
      for (int k = 0; k < p->num_refs; ++k) {
        shapes.push_back({p->refs[k].h, p->refs[k].w, p->refs[k].t_offset});
        lat.push_back(p->refs[k].latent);
      }
      flux_cuda_sampler *s = nullptr;
      note(res[r], flux_cuda_sampler_create(g->model[r], p->h, p->w, p->txt_seq, shapes.data(), p->num_refs, 1,
                                            p->num_steps, &s));
      for (int i = r; i < n_images && !res[r].rc; i += n) {
        note(res[r], flux_cuda_sampler_upload(s, z0[i], ctx[i], nullptr, lat.data()));
        if (!res[r].rc) note(res[r], flux_cuda_sampler_run(s, p->schedule, p->num_steps, 1.0f, 0, 1));
        if (!res[r].rc) note(res[r], flux_cuda_sampler_download(s, latent_out[i], nullptr));
      }
      flux_cuda_sampler_free(s);
    });
  for (auto &t : th)
    if (t.joinable()) t.join();
  for (int r = 0; r < n; ++r)
    if (res[r].rc) {
      set_error("GPU member %d: %s", r, res[r].msg.c_str());
      return res[r].rc;
    }
  return FLUX_CUDA_OK;
}

int flux_cuda_group_sample_cfg_pair(flux_cuda_group *g, const flux_cuda_sample_params *p, const float *z0,
                                    float *latent_out) {
  if (!g || !p || !z0 || !latent_out || !p->ctx || !p->ctx_uncond || !p->schedule || p->num_steps < 1) {
    set_error("group_sample_cfg_pair: bad argument (both contexts are needed)");
    return FLUX_CUDA_ERR_ARG;
  }
  if (g->ctx.size() < 2 || !g->peer_ok) {
    set_error("group_sample_cfg_pair: needs two GPUs that can reach each other's memory");
    return FLUX_CUDA_ERR_ARG;
  }
  if (!g->model[0] || !g->model[1]) {
    set_error("group: no model on the pair's members");
    return FLUX_CUDA_ERR_MODEL;
  }
  const size_t n_lat = static_cast<size_t>(g->model[0]->d.latent_ch) * p->h * p->w;
  int rc = pair_buffers(g, n_lat);
  if (rc) return rc;
  // a fresh rendezvous per image: a member that gave up in an earlier image must not poison this one
  flux_cuda_rendezvous_destroy(g->rv);
  g->rv = nullptr;
  rc = flux_cuda_rendezvous_create(2, &g->rv);
  if (rc) return rc;
  const int seq0 = g->seq;
  WorkerResult res[2];
  std::thread th[2];
  for (int r = 0; r < 2; ++r)
    if (!spawn(th[r], res[r], [&, r]() {
      flux_cuda_ctx *c = g->ctx[r];
      const int peer = r ^ 1;
      const float coef = r == 0 ? p->guidance : 1.0f - p->guidance;  // member 0 runs the conditional pass
      std::vector<flux_cuda_ref_shape> shapes;
      std::vector<const float *> lat;
      for (int k = 0; k < p->num_refs; ++k) {
        shapes.push_back({p->refs[k].h, p->refs[k].w, p->refs[k].t_offset});
        lat.push_back(p->refs[k].latent);
      }
      flux_cuda_sampler *s = nullptr;
      note(res[r], flux_cuda_sampler_create(g->model[r], p->h, p->w, p->txt_seq, shapes.data(), p->num_refs, 1,
                                            p->num_steps, &s));
      if (!res[r].rc) note(res[r], flux_cuda_sampler_upload(s, z0, r == 0 ? p->ctx : p->ctx_uncond, nullptr, lat.data()));
      for (int i = 0; i < p->num_steps && !res[r].rc; ++i) {
        note(res[r], flux_cuda_sampler_predict(s, p->schedule, p->num_steps, i));
        if (res[r].rc) break;
        // both host threads have queued this step's forward pass before either queues the kernel that waits
        note(res[r], flux_cuda_rendezvous_arrive_and_wait(g->rv, r, seq0 + i + 1, g->timeout_ms));
        if (res[r].rc) break;
        cudaSetDevice(c->device);
        const int slot = (seq0 + i) & 1;
        const int blocks = static_cast<int>((n_lat + 256 * 8 - 1) / (256 * 8)) < 64
                               ? static_cast<int>((n_lat + 256 * 8 - 1) / (256 * 8))
                               : 64;
        pair_exchange_euler_kernel<<<blocks, 256, 0, c->stream>>>(
            s->ws->z, s->ws->v, coef, s->ws->sched, i, static_cast<long long>(n_lat),
            g->inbox[peer] + static_cast<size_t>(slot) * g->inbox_floats, g->flag[peer],
            g->inbox[r] + static_cast<size_t>(slot) * g->inbox_floats, g->flag[r], g->counter[r], seq0 + i + 1,
            c->err_dev, WAIT_LIMIT_CYCLES);
        note(res[r], check_cuda(cudaGetLastError(), "pair exchange launch"));
      }
      if (res[r].rc) flux_cuda_rendezvous_abandon(g->rv, r);
      // member 0 returns the latent; member 1 only waits for its queue and reports kernel errors
      if (s) note(res[r], flux_cuda_sampler_download(s, r == 0 ? latent_out : nullptr, nullptr));
      flux_cuda_sampler_free(s);
    }))
      flux_cuda_rendezvous_abandon(g->rv, r);  // the other member must not wait for a thread that never started
  for (int r = 0; r < 2; ++r)
    if (th[r].joinable()) th[r].join();
  g->seq = seq0 + p->num_steps;
  for (int r = 0; r < 2; ++r)
    if (res[r].rc) {
      set_error("GPU member %d: %s", r, res[r].msg.c_str());
      return res[r].rc;
    }
  return FLUX_CUDA_OK;
}

}  // extern "C"
