// Worker-pool request scheduler over shared-weight contexts (see scheduler.hpp).
#include "scheduler.hpp"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <thread>

#include "../common.cuh"

namespace evob {

double log_probability(const float *logits, const std::size_t vocab, const std::size_t target) {
  float maximum = logits[0];
  for (std::size_t i = 1; i < vocab; ++i) maximum = std::max(maximum, logits[i]);
  double total = 0.0;
  for (std::size_t i = 0; i < vocab; ++i)
    total += std::exp(static_cast<double>(logits[i]) - static_cast<double>(maximum));
  return static_cast<double>(logits[target]) - static_cast<double>(maximum) - std::log(total);
}

struct Scheduler::Impl {
  struct Work {
    std::uint64_t ticket = 0;
    SchedulerRequest request;
    Completion done;
    std::atomic<bool> cancelled{false};
    std::chrono::steady_clock::time_point submitted;
  };

  std::shared_ptr<ModelWeights> weights;
  std::vector<std::unique_ptr<Context>> contexts;
  std::vector<std::thread> threads;
  std::size_t maximum_queue = 0, context_size = 0;
  ExecutionProfile profile = ExecutionProfile::kExact;
  bool full_arena = false, q8_kv = false;

  mutable std::mutex mutex;
  mutable std::condition_variable wake, idle;
  std::deque<std::shared_ptr<Work>> pending;
  std::map<std::uint64_t, std::shared_ptr<Work>> live;  // queued or running, by ticket
  std::uint64_t next_ticket = 1;
  bool stopping = false;
  SchedulerMetrics counters;

  // One request on the worker's own context.  The context is reusable: an
  // initial prefill resets every cache; a context that a failure has retired is
  // replaced before the next request.
  void run(Context &context, Work &work, SchedulerResult *result) {
    const SchedulerRequest &request = work.request;
    const std::size_t vocab = context.config().vocab;
    const std::size_t chunk = context.activation_capacity();
    const std::vector<std::uint8_t> &bytes = request.sequence;
    const bool score = request.kind == SchedulerRequest::Kind::kScore;
    if (bytes.empty() || (score && bytes.size() < 2)) {
      result->status = kInvalidArgument;
      result->error = score ? "scoring needs at least two tokens" : "generation needs a prompt";
      return;
    }
    if (bytes.size() + (score ? 0 : request.new_tokens) > context.context_capacity()) {
      result->status = kInvalidArgument;
      result->error = "request exceeds the context capacity of " + std::to_string(context.context_capacity());
      return;
    }
    if (!score && validate_sampling(request.sampling) != kOk) {
      result->status = kInvalidArgument;
      result->error = last_error();
      return;
    }
    std::vector<float> logits;
    std::vector<std::uint32_t> tokens;
    for (std::size_t offset = 0; offset < bytes.size(); offset += chunk) {
      if (work.cancelled.load(std::memory_order_relaxed)) {
        result->cancelled = true;
        return;
      }
      const std::size_t rows = std::min(chunk, bytes.size() - offset);
      tokens.assign(bytes.begin() + static_cast<std::ptrdiff_t>(offset),
                    bytes.begin() + static_cast<std::ptrdiff_t>(offset + rows));
      const int status = offset == 0 ? context.prefill(tokens, &logits) : context.prefill_chunk(tokens, &logits);
      if (status != kOk) {
        result->status = status;
        result->error = last_error();
        return;
      }
      if (score) {
        // row r of this chunk predicts byte offset + r + 1
        for (std::size_t r = 0; r < rows && offset + r + 1 < bytes.size(); ++r) {
          const double value = log_probability(logits.data() + r * vocab, vocab, bytes[offset + r + 1]);
          result->token_log_likelihoods.push_back(value);
          result->log_likelihood += value;
        }
      }
    }
    if (score) {
      result->scored_tokens = bytes.size() - 1;
      return;
    }
    Sampler sampler(request.sampling);
    const float *last_row = logits.data() + (logits.size() / vocab - 1) * vocab;
    std::vector<float> step;
    for (std::size_t produced = 0; produced < request.new_tokens; ++produced) {
      if (work.cancelled.load(std::memory_order_relaxed)) {
        result->cancelled = true;
        return;
      }
      std::uint32_t token = 0;
      int status = sampler.sample(last_row, vocab, &token);
      if (status == kOk && token > 255) break;  // not a byte: generation ends (upstream token_to_byte)
      if (status == kOk) {
        result->generated.push_back(static_cast<std::uint8_t>(token));
        if (produced + 1 == request.new_tokens) break;
        status = context.decode(token, &step);
      }
      if (status != kOk) {
        result->status = status;
        result->error = last_error();
        return;
      }
      last_row = step.data();
    }
  }

  void worker(const std::size_t index) {
    for (;;) {
      std::shared_ptr<Work> work;
      {
        std::unique_lock<std::mutex> lock(mutex);
        wake.wait(lock, [&] { return stopping || !pending.empty(); });
        if (pending.empty()) return;  // stopping and drained
        work = std::move(pending.front());
        pending.pop_front();
        counters.queued = pending.size();
        ++counters.active;
        counters.active_peak = std::max(counters.active_peak, counters.active);
      }
      SchedulerResult result;
      const auto begin = std::chrono::steady_clock::now();
      result.queue_seconds = std::chrono::duration<double>(begin - work->submitted).count();
      if (work->cancelled.load(std::memory_order_relaxed)) {
        result.cancelled = true;
      } else {
        try {
          if (contexts[index] == nullptr || contexts[index]->poisoned()) {
            contexts[index].reset();
            const int status = Context::create(weights, context_size, profile, full_arena, &contexts[index], q8_kv);
            if (status != kOk) {
              result.status = status;
              result.error = last_error();
            }
          }
          if (result.status == kOk) run(*contexts[index], *work, &result);
        } catch (const std::exception &error) {
          result.status = kInternal;
          result.error = error.what();
        } catch (...) {
          result.status = kInternal;
          result.error = "scheduler task threw";
        }
      }
      result.run_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - begin).count();
      if (work->done) {
        try {
          work->done(work->ticket, result);
        } catch (...) {
        }
      }
      {
        std::lock_guard<std::mutex> lock(mutex);
        --counters.active;
        if (result.cancelled) ++counters.cancelled;
        else if (result.status != kOk) ++counters.failed;
        else ++counters.completed;
        live.erase(work->ticket);
        if (pending.empty() && counters.active == 0) idle.notify_all();
      }
    }
  }
};

int Scheduler::create(std::shared_ptr<ModelWeights> weights, const std::size_t workers,
                      const std::size_t maximum_queue, const std::size_t context_size,
                      const ExecutionProfile profile, const bool full_arena_for_fixtures, const bool q8_kv,
                      std::unique_ptr<Scheduler> *out) {
  if (out == nullptr || weights == nullptr || workers == 0 || workers > 64 || maximum_queue == 0 ||
      maximum_queue < workers || context_size == 0)
    return fail(kInvalidArgument, "invalid dynamic scheduler limits");
  if (weights->slice_count > 1)
    return fail(kInvalidArgument, "a scheduler needs a whole model, not one pipeline slice");
  std::unique_ptr<Scheduler> scheduler(new Scheduler());
  scheduler->impl_ = std::make_unique<Impl>();
  Impl &impl = *scheduler->impl_;
  impl.weights = std::move(weights);
  impl.maximum_queue = maximum_queue;
  impl.context_size = context_size;
  impl.profile = profile;
  impl.full_arena = full_arena_for_fixtures;
  impl.q8_kv = q8_kv;
  impl.contexts.resize(workers);
  for (std::size_t i = 0; i < workers; ++i) {
    const int status = Context::create(impl.weights, context_size, profile, full_arena_for_fixtures,
                                       &impl.contexts[i], q8_kv);
    if (status != kOk) return status;
  }
  for (std::size_t i = 0; i < workers; ++i) impl.threads.emplace_back([&impl, i] { impl.worker(i); });
  *out = std::move(scheduler);
  return kOk;
}

Scheduler::~Scheduler() {
  if (impl_ == nullptr) return;
  {
    std::lock_guard<std::mutex> lock(impl_->mutex);
    impl_->stopping = true;
    for (auto &entry : impl_->live) entry.second->cancelled.store(true, std::memory_order_relaxed);
  }
  impl_->wake.notify_all();
  for (std::thread &thread : impl_->threads)
    if (thread.joinable()) thread.join();
}

std::uint64_t Scheduler::submit(SchedulerRequest request, Completion done) {
  auto work = std::make_shared<Impl::Work>();
  work->request = std::move(request);
  work->done = std::move(done);
  work->submitted = std::chrono::steady_clock::now();
  {
    std::lock_guard<std::mutex> lock(impl_->mutex);
    if (impl_->stopping || impl_->pending.size() >= impl_->maximum_queue) {
      ++impl_->counters.rejected;
      return 0;
    }
    work->ticket = impl_->next_ticket++;
    impl_->pending.push_back(work);
    impl_->live[work->ticket] = work;
    ++impl_->counters.submitted;
    impl_->counters.queued = impl_->pending.size();
    impl_->counters.queue_peak = std::max(impl_->counters.queue_peak, impl_->counters.queued);
  }
  impl_->wake.notify_one();
  return work->ticket;
}

bool Scheduler::cancel(const std::uint64_t ticket) {
  std::lock_guard<std::mutex> lock(impl_->mutex);
  const auto found = impl_->live.find(ticket);
  if (found == impl_->live.end()) return false;
  found->second->cancelled.store(true, std::memory_order_relaxed);
  return true;
}

SchedulerMetrics Scheduler::metrics() const {
  std::lock_guard<std::mutex> lock(impl_->mutex);
  return impl_->counters;
}

void Scheduler::wait_idle() const {
  std::unique_lock<std::mutex> lock(impl_->mutex);
  impl_->idle.wait(lock, [&] { return impl_->pending.empty() && impl_->counters.active == 0; });
}

}  // namespace evob
