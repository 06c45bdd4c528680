// Host-side expert arithmetic for the CPU expert service: a persistent thread pool (workers optionally pinned to a CPU
// list, e.g. the cores of one NUMA node) and NVFP4 linears that read the checkpoint's packed form directly.
//
// NVFP4: E2M1 codes, two per byte (low nibble = even k), one E4M3 scale per 16 elements, one fp32 tensor scale. The
// weights stay packed in host memory (4.5 bits per weight: a token's routed experts stream 7x fewer bytes than fp32
// copies would), a 16-element block is decoded with one byte shuffle (codes doubled so that they are integers:
// 0 1 2 3 4 6 8 12), multiplied with the activations in fp32 and scaled once per block.
// The AVX2 + FMA path is chosen at run time; the scalar path is the statement of the same sums.
// One expert on one row: out += weight * bf16(down(bf16(act(gate) * up))) with gate | up = bf16(W_gu x): the rounding
// points of the device path, so a route computed here matches a route computed on the GPU to summation order.
// Reference counterpart: src/kernels/cpu/nvfp4_linear.cpp, src/kernels/cpu/pool.cpp, src/runtime/cpu_expert_pool.cpp.
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif
#if defined(__linux__)
#include <pthread.h>
#include <sched.h>
#endif

namespace {

struct Pool {
  std::vector<std::thread> workers;
  std::mutex m;
  std::condition_variable cv, done_cv;
  std::function<void(int, int)> job;
  uint64_t generation = 0;
  int pending = 0;
  bool stop = false;
  int spin_us = 0;
  std::atomic<uint64_t> gen_atomic{0};

  void worker(int id, int n, int cpu) {
#if defined(__linux__)
    if (cpu >= 0) {
      cpu_set_t set;
      CPU_ZERO(&set);
      CPU_SET(cpu, &set);
      pthread_setaffinity_np(pthread_self(), sizeof(set), &set);      // best effort: a refused mask leaves the thread floating
    }
#endif
    uint64_t seen = 0;
    for (;;) {
      // spin for a while on the generation counter (a decode step posts work every few hundred microseconds), then sleep
      if (spin_us > 0) {
        const auto t0 = std::chrono::steady_clock::now();
        while (gen_atomic.load(std::memory_order_acquire) == seen &&
               std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count() < spin_us) {
#if defined(__x86_64__)
          _mm_pause();
#endif
        }
      }
      std::function<void(int, int)> fn;
      {
        std::unique_lock<std::mutex> lk(m);
        cv.wait(lk, [&] { return stop || generation != seen; });
        if (stop) return;
        seen = generation;
        fn = job;
      }
      fn(id, n);
      {
        std::lock_guard<std::mutex> lk(m);
        if (--pending == 0) done_cv.notify_all();
      }
    }
  }

  void run(const std::function<void(int, int)>& fn) {
    const int n = (int)workers.size();
    if (n == 0) {
      fn(0, 1);
      return;
    }
    {
      std::lock_guard<std::mutex> lk(m);
      job = fn;
      pending = n;
      ++generation;
      gen_atomic.store(generation, std::memory_order_release);
    }
    cv.notify_all();
    std::unique_lock<std::mutex> lk(m);
    done_cv.wait(lk, [&] { return pending == 0; });
  }
};

float e4m3_table[256];
std::once_flag table_once;
void init_tables() {
  for (int b = 0; b < 256; ++b) {
    const int s = b >> 7, e = (b >> 3) & 15, mnt = b & 7;
    float v;
    if (e == 0) v = std::ldexp((float)mnt / 8.f, -6);
    else if (e == 15 && mnt == 7) v = NAN;
    else v = std::ldexp(1.f + (float)mnt / 8.f, e - 7);
    e4m3_table[b] = s ? -v : v;
  }
}

// doubled E2M1 values: code bits [sign | exp exp | man]
const int8_t kE2M1x2[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

inline float bf16_round(float v) {
  uint32_t u;
  std::memcpy(&u, &v, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return v;
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  std::memcpy(&v, &u, 4);
  return v;
}

float dot_row_scalar(const uint8_t* w, const uint8_t* sc, const float* x, int K) {
  float acc = 0.f;
  for (int b = 0; b < K / 16; ++b) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) {
      const uint8_t byte = w[b * 8 + i];
      s += (float)kE2M1x2[byte & 15] * x[b * 16 + 2 * i] + (float)kE2M1x2[byte >> 4] * x[b * 16 + 2 * i + 1];
    }
    acc += s * e4m3_table[sc[b]];
  }
  return 0.5f * acc;
}

#if defined(__x86_64__)
__attribute__((target("avx2,fma"))) float dot_row_avx2(const uint8_t* w, const uint8_t* sc, const float* x, int K) {
  const __m128i lut = _mm_loadu_si128(reinterpret_cast<const __m128i*>(kE2M1x2));
  const __m128i m4 = _mm_set1_epi8(0x0f);
  __m256 acc = _mm256_setzero_ps();
  for (int b = 0; b < K / 16; ++b) {
    const __m128i raw = _mm_loadl_epi64(reinterpret_cast<const __m128i*>(w + b * 8));
    const __m128i lo = _mm_shuffle_epi8(lut, _mm_and_si128(raw, m4));
    const __m128i hi = _mm_shuffle_epi8(lut, _mm_and_si128(_mm_srli_epi16(raw, 4), m4));
    const __m128i v = _mm_unpacklo_epi8(lo, hi);                       // 16 codes in element order
    const __m256 f0 = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(v));
    const __m256 f1 = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_srli_si128(v, 8)));
    __m256 s = _mm256_mul_ps(f0, _mm256_loadu_ps(x + b * 16));
    s = _mm256_fmadd_ps(f1, _mm256_loadu_ps(x + b * 16 + 8), s);
    acc = _mm256_fmadd_ps(s, _mm256_set1_ps(e4m3_table[sc[b]]), acc);
  }
  __m128 r = _mm_add_ps(_mm256_castps256_ps128(acc), _mm256_extractf128_ps(acc, 1));
  r = _mm_add_ps(r, _mm_movehl_ps(r, r));
  r = _mm_add_ss(r, _mm_shuffle_ps(r, r, 1));
  return 0.5f * _mm_cvtss_f32(r);
}
#endif

bool use_avx2() {
#if defined(__x86_64__)
  static const bool ok = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
  return ok;
#else
  return false;
#endif
}

inline float dot_row(const uint8_t* w, const uint8_t* sc, const float* x, int K) {
#if defined(__x86_64__)
  if (use_avx2()) return dot_row_avx2(w, sc, x, K);
#endif
  return dot_row_scalar(w, sc, x, K);
}

void gemv(Pool* pool, const uint8_t* packed, const uint8_t* scales, float gscale, const float* x, float* y, int N, int K) {
  auto body = [&](int id, int n) {
    const int per = (N + n - 1) / n, lo = id * per, hi = std::min(N, lo + per);
    for (int r = lo; r < hi; ++r) y[r] = gscale * dot_row(packed + (size_t)r * (K / 2), scales + (size_t)r * (K / 16), x, K);
  };
  if (pool) pool->run(body);
  else body(0, 1);
}

}  // namespace

extern "C" {

// threads <= 0: no workers (calls run on the caller's thread). cpus: optional list the workers are pinned to, round robin.
void* vh_cpu_pool_create(int threads, const int* cpus, int n_cpus, int spin_us) {
  std::call_once(table_once, init_tables);
  Pool* p = new Pool();
  p->spin_us = spin_us;
  for (int i = 0; i < threads; ++i) {
    const int cpu = (cpus && n_cpus > 0) ? cpus[i % n_cpus] : -1;
    p->workers.emplace_back([p, i, threads, cpu] { p->worker(i, threads, cpu); });
  }
  return p;
}

void vh_cpu_pool_destroy(void* h) {
  Pool* p = static_cast<Pool*>(h);
  if (!p) return;
  {
    std::lock_guard<std::mutex> lk(p->m);
    p->stop = true;
  }
  p->cv.notify_all();
  for (auto& t : p->workers) t.join();
  delete p;
}

int vh_cpu_pool_threads(void* h) { return h ? (int)static_cast<Pool*>(h)->workers.size() : 0; }
int vh_cpu_has_avx2() { return use_avx2() ? 1 : 0; }

// y[n] = gscale * sum_k W[n, k] x[k]. packed [N, K / 2], scales [N, K / 16] (E4M3 bytes, row major), K % 16 == 0.
int vh_cpu_nvfp4_gemv(void* pool, const void* packed, const void* scales, float gscale, const float* x, float* y, int N, int K) {
  std::call_once(table_once, init_tables);
  if (N <= 0 || K <= 0 || K % 16) return 1;
  gemv(static_cast<Pool*>(pool), (const uint8_t*)packed, (const uint8_t*)scales, gscale, x, y, N, K);
  return 0;
}

// out[h] += weight * bf16(W_dn a), a = bf16(act(g) * u), [g | u] = bf16(W_gu x): one routed expert on one row.
// W_gu [2 I, H] (gate rows then up rows), W_dn [H, I]; act 0 SiLU, 1 tanh GELU; limit > 0 clamps g from above and u to
// [-limit, limit]. scratch: 3 I floats.
int vh_cpu_nvfp4_expert(void* pool, const void* gu_packed, const void* gu_scales, float gu_g, const void* dn_packed,
                        const void* dn_scales, float dn_g, const float* x, float* out, int H, int I, int act, float limit,
                        float weight, float* scratch) {
  std::call_once(table_once, init_tables);
  if (H <= 0 || I <= 0 || H % 16 || I % 16 || !scratch) return 1;
  Pool* p = static_cast<Pool*>(pool);
  float* gu = scratch;            // [2 I]
  float* a = scratch + 2 * I;     // [I]
  gemv(p, (const uint8_t*)gu_packed, (const uint8_t*)gu_scales, gu_g, x, gu, 2 * I, H);
  for (int i = 0; i < I; ++i) {
    float g = bf16_round(gu[i]), u = bf16_round(gu[I + i]);
    if (limit > 0.f) {
      g = std::min(g, limit);
      u = std::max(-limit, std::min(u, limit));
    }
    const float t = act == 0 ? g / (1.f + std::exp(-g))
                             : 0.5f * g * (1.f + std::tanh(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    a[i] = bf16_round(t * u);
  }
  std::vector<float> y((size_t)H);
  gemv(p, (const uint8_t*)dn_packed, (const uint8_t*)dn_scales, dn_g, a, y.data(), H, I);
  for (int h = 0; h < H; ++h) out[h] += weight * bf16_round(y[h]);
  return 0;
}

}  // extern "C"
