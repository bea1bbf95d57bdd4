// Request scheduler over shared-weight contexts of one model: the serving
// loop behind upstream's `evo serve` (DynamicScheduler, include/evo/server.hpp:
// 59-88 and src/scheduler.cpp:49-201, driven from src/server.cpp) without its
// HTTP transport.
//
// Upstream collects up to `maximum_batch` queued tasks inside a batch window,
// starts one thread per task, and joins them all before it looks at the queue
// again, so a short request waits for the longest one of its batch and every
// request builds its own context.  Here `workers` threads each own one
// long-lived context of the model (own stream, arena and caches; immutable
// weights shared, as upstream's initialize_shared does,
// src/cuda/model.cu:2596-2691) and pull requests as they become free: no batch
// barrier and no per-request allocation.  Kernels of different contexts overlap
// on the GPU wherever one request alone leaves SMs idle (short prompts,
// decode).  Kept from upstream: a bounded queue that refuses new work when
// full, cancellation before and between steps, and the metrics counters.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "model.hpp"
#include "sampler.hpp"

namespace evob {

struct SchedulerRequest {
  enum class Kind { kScore, kGenerate };
  Kind kind = Kind::kScore;
  std::vector<std::uint8_t> sequence;  // bytes to score, or the prompt
  std::size_t new_tokens = 0;          // generate: tokens to sample after the prompt
  SamplingConfig sampling;
};

struct SchedulerResult {
  int status = 0;                   // evo_status of the request (0 = ok)
  std::string error;                // message when status != kOk
  bool cancelled = false;
  double log_likelihood = 0.0;      // score: sum of next-token log-likelihoods
  std::size_t scored_tokens = 0;
  std::vector<double> token_log_likelihoods;
  std::vector<std::uint8_t> generated;  // generate: sampled bytes (stops early at a token above 255)
  double queue_seconds = 0.0, run_seconds = 0.0;
};

struct SchedulerMetrics {
  std::uint64_t submitted = 0, rejected = 0, completed = 0, failed = 0, cancelled = 0;
  std::size_t queued = 0, queue_peak = 0, active = 0, active_peak = 0;
};

class Scheduler {
 public:
  using Completion = std::function<void(std::uint64_t ticket, const SchedulerResult &result)>;

  // `workers` contexts of `context_size` tokens are created up front.
  static int create(std::shared_ptr<ModelWeights> weights, std::size_t workers, std::size_t maximum_queue,
                    std::size_t context_size, ExecutionProfile profile, bool full_arena_for_fixtures,
                    bool q8_kv, std::unique_ptr<Scheduler> *out);
  ~Scheduler();  // cancels what is queued, lets running requests finish their current step, joins

  // 0 when the queue is full or the scheduler is stopping (counted as rejected);
  // otherwise the ticket that `done` will be called with, on a worker thread.
  std::uint64_t submit(SchedulerRequest request, Completion done);
  // Marks a queued or running request; it completes with cancelled = true at its next check.
  bool cancel(std::uint64_t ticket);
  SchedulerMetrics metrics() const;
  void wait_idle() const;  // until nothing is queued or running

 private:
  struct Impl;
  Scheduler() = default;
  std::unique_ptr<Impl> impl_;
};

// log softmax(logits)[target] in double, summed in index order: the scoring
// rule of upstream's drivers (src/cuda/inference_cli.cpp:199-224).
double log_probability(const float *logits, std::size_t vocab, std::size_t target);

}  // namespace evob
