// Drop-in replacement for the reference's getp-csrc/getp_run.cpp on NVIDIA B200: defines the three functions
// the fixed harness getp-csrc/getp_eval.cpp declares and calls (getp_eval.cpp:97-145) —
//     void warm_up(Transformer *, Tokenizer *);
//     long long inference(Transformer *, Tokenizer *, Sampler *, Requests *);
//     void finish(Transformer *, Tokenizer *);
// — on top of the gptoss_b200 C ABI.  Like the file it replaces it is textually included by run.cpp
// (run.cpp:1071-1072), so it sees the reference's Transformer/Config (run.cpp:25-117), Requests
// (getp_eval.cpp:9-15) and encode() (tokenizer.hpp:45).
//
// Scheduling follows the reference's 20B engine (getp-csrc/submit/getp_run_submit.cpp:4-104): requests are
// cut into batches, each batch decodes in lock-step from position 0, prompt tokens are force-fed one per
// step, the first generated token lands at index 0 of the request's output row, a sequence stops at the
// end-of-sequence ids 199999 / 200002, and each output row is terminated by -1 after generated_len + 1 ids.
// Batches are spread over the GPUs (GPTOSS_GPUS, default 1) as data-parallel replicas, one host thread and one
// model per GPU (DP_20B, getp-csrc/include/config.hpp:16-19).  With GPTOSS_EP=1 the GPUs instead decode every
// batch together, like the reference's 120B engine (forward_gpu_120b_batched, getp-csrc/src/model.cpp:153-489; one
// host thread per GPU meeting at a pthread barrier, getp-csrc/getp_run.cpp): the experts are sharded over the GPUs,
// the sequences of a batch are dealt out in slices, and the ranks exchange activations over peer memory on the
// device.  Batch size: environment GPTOSS_BATCH (default 1024; with GPTOSS_EP the batch of the whole group).
//
// Beyond the reference's scheduler (which keeps stepping a finished sequence until its whole batch has drained,
// getp_run_submit.cpp:60-96): a data-parallel replica drops finished sequences from its batch between steps.  The
// survivors keep their KV-cache rows (gptoss_model_step_rows takes the row of each live sequence), nothing is copied,
// and since a sequence's tokens do not depend on its batch mates the output is unchanged; GPTOSS_NO_COMPACT=1 switches
// it off.  GPTOSS_STOP_IDS="id,id,..." names further token ids that end a sequence like 199999 / 200002 do.
// By default a replica goes one step further and batches continuously: it holds GPTOSS_BATCH slots, and a slot whose
// sequence has finished is handed to the next waiting request at once, which starts at position 0 while the other
// slots carry on (gptoss_model_step_seqs takes a position per sequence); the replicas draw requests from one queue.
// Each request's tokens are what the batch-at-a-time schedule produces.  GPTOSS_NO_CONTINUOUS=1 restores that schedule.
#include "getp_eval.cpp"

#include <pthread.h>

#include <algorithm>
#include <atomic>
#include <thread>
#include <vector>

extern "C" {
#include "gptoss_b200.h"
}

#ifndef GETP_RUN
#define GETP_RUN

namespace {

std::vector<gptoss_model *> g_models;  // one per GPU
int g_batch = 1024;
int g_max_seq = 0;
bool g_group = false;  // GPTOSS_EP: the models are the ranks of one group
bool g_compact = true;  // drop finished sequences from a replica's batch between steps
bool g_continuous = true;  // refill a finished sequence's slot with the next request instead of draining the batch
std::vector<int> g_stop_ids = {199999, 200002};  // run.cpp:939, getp_run_submit.cpp:249

bool is_stop(int tok) { return std::find(g_stop_ids.begin(), g_stop_ids.end(), tok) != g_stop_ids.end(); }

void die(const char *what, gptoss_model *m) {
  fprintf(stderr, "gptoss_b200: %s: %s\n", what, m ? gptoss_model_last_error(m) : "");
  exit(EXIT_FAILURE);
}

gptoss_model_config to_config(const Config &c) {
  gptoss_model_config g;
  static_assert(sizeof(gptoss_model_config) == sizeof(Config), "checkpoint header layout");
  memcpy(&g, &c, sizeof g);
  return g;
}

// What the ranks of a group agree on after every step: how many sequences are still running anywhere.
struct GroupSync {
  pthread_barrier_t bar;
  std::vector<int> active;  // per rank
  explicit GroupSync(int ranks) : active(ranks, 0) { pthread_barrier_init(&bar, nullptr, ranks); }
  ~GroupSync() { pthread_barrier_destroy(&bar); }
  int total_active(int rank, int mine) {
    active[rank] = mine;
    pthread_barrier_wait(&bar);
    int t = 0;
    for (int a : active) t += a;
    pthread_barrier_wait(&bar);  // nobody overwrites its entry before everyone has read it
    return t;
  }
};

std::vector<int> encode_prompt(Tokenizer *tokenizer, const Config &cfg, Requests *reqs, int idx) {
  const char *text = get_str_req_ptr(reqs, idx);
  std::vector<int> buf(strlen(text) + 3);
  int count = 0;
  encode(tokenizer, text, -1, -1, buf.data(), &count, cfg.initial_context_length);
  if (count < 1) {
    fprintf(stderr, "something is wrong, expected at least 1 prompt token\n");
    exit(EXIT_FAILURE);
  }
  buf.resize(count);
  return buf;
}

// One batch of requests [first, first + n) in lock-step.  Returns the token count the reference reports
// (generated_len + 1 per request).  A single model decodes the whole batch; a rank of a group (sync != nullptr) its
// slice of it, and keeps stepping, for the other ranks' sake, until no sequence of the batch is running anywhere.
long long run_batch(gptoss_model *model, Tokenizer *tokenizer, const Config &cfg, Requests *reqs, int first, int n,
                    GroupSync *sync = nullptr, int rank = 0) {
  const int max_seq_len = reqs->max_seq_len;
  const int batch = n;  // the batch of the whole group
  if (sync) {
    int s_first = 0, s_n = 0;
    gptoss_model_slice(model, batch, &s_first, &s_n);
    first += s_first;
    n = s_n;
  }
  std::vector<std::vector<int>> prompt(n);
  for (int i = 0; i < n; ++i) prompt[i] = encode_prompt(tokenizer, cfg, reqs, first + i);
  std::vector<int> cur(n), next(n), pos_of(n, 0);
  std::vector<char> active(n, 1);
  int n_active = n;
  for (int i = 0; i < n; ++i) cur[i] = prompt[i][0];
  int running = sync ? sync->total_active(rank, n_active) : n_active;
  const bool compact = g_compact && !sync;  // the ranks of a group keep their slices
  std::vector<int> live, cur_live, next_live;  // compacted batch: sequence indices (= KV-cache rows), inputs, outputs
  for (int pos = 0; pos < max_seq_len - 1 && running > 0; ++pos) {
    bool need_next = false;  // does any running sequence take the model's token this step?
    for (int i = 0; i < n && !need_next; ++i) need_next = active[i] && pos_of[i] >= (int)prompt[i].size() - 1;
    if (compact && n_active < n) {
      if ((int)live.size() != n_active) {  // somebody finished since the last step
        live.clear();
        for (int i = 0; i < n; ++i)
          if (active[i]) live.push_back(i);
        cur_live.resize(live.size());
        next_live.resize(live.size());
      }
      for (size_t j = 0; j < live.size(); ++j) cur_live[j] = cur[live[j]];
      if (gptoss_model_step_rows(model, cur_live.data(), live.data(), pos, (int)live.size(), need_next ? next_live.data() : nullptr))
        die("decode step failed", model);
      for (size_t j = 0; j < live.size(); ++j) next[live[j]] = next_live[j];
    } else if (gptoss_model_step(model, cur.data(), pos, batch, need_next ? next.data() : nullptr)) {
      die("decode step failed", model);
    }
    for (int i = 0; i < n; ++i) {
      if (!active[i]) continue;
      int tok = next[i];
      const int n_prompt = (int)prompt[i].size();
      if (pos_of[i] < n_prompt - 1)
        tok = prompt[i][pos_of[i] + 1];  // still inside the prompt: force-feed
      else
        get_tok_gen_ptr(reqs, first + i)[pos_of[i] - (n_prompt - 1)] = tok;
      if (is_stop(tok)) {
        active[i] = 0;
        --n_active;
      }
      cur[i] = tok;
      ++pos_of[i];
    }
    running = sync ? sync->total_active(rank, n_active) : n_active;
  }
  long long count = 0;
  for (int i = 0; i < n; ++i) {
    const int generated_len = std::max(0, pos_of[i] - (int)prompt[i].size());
    get_tok_gen_ptr(reqs, first + i)[generated_len + 1] = -1;
    count += generated_len + 1;
  }
  return count;
}

// Continuous batching on one replica: `g_batch` slots (slot s = KV-cache row s), requests drawn from the shared queue
// `next_req` whenever a slot is free.  Per sequence the rules are those of run_batch: prompt tokens force-fed one per
// step, generated tokens from index 0 of the request's output row, stop ids, at most max_seq_len - 1 steps, the row
// terminated by -1 after generated_len + 1 ids.
long long run_continuous(gptoss_model *model, Tokenizer *tokenizer, const Config &cfg, Requests *reqs, std::atomic<int> &next_req) {
  struct Slot {
    int req = -1;  // request index, -1 = free
    std::vector<int> prompt;
    int pos = 0, cur = 0;
  };
  const int max_seq_len = reqs->max_seq_len;
  std::vector<Slot> slots(g_batch);
  std::vector<int> tokens, rows, pos, next;
  long long count = 0;
  bool queue_empty = max_seq_len < 2;  // no step fits: nothing is taken from the queue (run_batch would write -1 only)
  if (queue_empty) {
    for (int r = next_req++; r < reqs->num_reqs; r = next_req++) {
      get_tok_gen_ptr(reqs, r)[1] = -1;
      ++count;
    }
    return count;
  }
  for (;;) {
    tokens.clear(), rows.clear(), pos.clear();
    bool need_next = false;
    for (int s = 0; s < g_batch; ++s) {
      Slot &sl = slots[s];
      if (sl.req < 0 && !queue_empty) {
        const int r = next_req++;
        if (r >= reqs->num_reqs) {
          queue_empty = true;
        } else {
          sl.req = r;
          sl.prompt = encode_prompt(tokenizer, cfg, reqs, r);
          sl.pos = 0;
          sl.cur = sl.prompt[0];
        }
      }
      if (sl.req < 0) continue;
      tokens.push_back(sl.cur), rows.push_back(s), pos.push_back(sl.pos);
      need_next = need_next || sl.pos >= (int)sl.prompt.size() - 1;
    }
    if (tokens.empty()) break;
    next.resize(tokens.size());
    if (gptoss_model_step_seqs(model, tokens.data(), rows.data(), pos.data(), (int)tokens.size(), need_next ? next.data() : nullptr))
      die("decode step failed", model);
    for (size_t j = 0; j < rows.size(); ++j) {
      Slot &sl = slots[rows[j]];
      const int n_prompt = (int)sl.prompt.size();
      int tok;
      if (sl.pos < n_prompt - 1)
        tok = sl.prompt[sl.pos + 1];  // still inside the prompt: force-feed
      else
        get_tok_gen_ptr(reqs, sl.req)[sl.pos - (n_prompt - 1)] = tok = next[j];
      sl.cur = tok;
      ++sl.pos;
      if (is_stop(tok) || sl.pos >= max_seq_len - 1) {
        const int generated_len = std::max(0, sl.pos - n_prompt);
        get_tok_gen_ptr(reqs, sl.req)[generated_len + 1] = -1;
        count += generated_len + 1;
        sl.req = -1;  // refilled at the top of the next step
      }
    }
  }
  return count;
}

}  // namespace

void warm_up(Transformer *transformer, Tokenizer *tokenizer) {
  (void)tokenizer;
  if (const char *b = getenv("GPTOSS_BATCH")) g_batch = std::max(1, atoi(b));
  int n_gpus = 1;
  if (const char *g = getenv("GPTOSS_GPUS")) n_gpus = std::max(1, atoi(g));
  if (const char *e = getenv("GPTOSS_EP")) g_group = atoi(e) != 0 && n_gpus > 1;
  if (const char *e = getenv("GPTOSS_NO_COMPACT")) g_compact = atoi(e) == 0;
  if (const char *e = getenv("GPTOSS_NO_CONTINUOUS")) g_continuous = atoi(e) == 0;
  if (const char *e = getenv("GPTOSS_STOP_IDS"))
    for (const char *p = e; *p;) {
      char *end = nullptr;
      const long v = strtol(p, &end, 10);
      if (end == p) break;
      g_stop_ids.push_back((int)v);
      p = *end ? end + 1 : end;
    }
  const Config &c = transformer->config;
  g_max_seq = c.seq_len;
  if (const char *s = getenv("GPTOSS_MAX_SEQ")) g_max_seq = std::min(c.seq_len, std::max(2, atoi(s)));
  const gptoss_model_config gc = to_config(c);
  for (int g = 0; g < n_gpus; ++g) {
    gptoss_model *m = nullptr;
    const int rc = g_group ? gptoss_model_create_ep(&gc, g, g, n_gpus, g_batch, g_max_seq, &m)
                           : gptoss_model_create(&gc, g, g_batch, g_max_seq, &m);
    if (rc) die("cannot create the model (GPU count, memory, dimensions, experts not divisible by the GPUs)", nullptr);
    // the reference keeps the whole file mapped: header first, then the tensors (run.cpp:274-280)
    if (gptoss_model_load_mem(m, transformer->data, (uint64_t)transformer->file_size)) die("cannot load the checkpoint", m);
    g_models.push_back(m);
  }
  if (g_group) {  // every rank maps every rank's exchange buffers
    std::vector<gptoss_ctx *> ctxs;
    for (gptoss_model *m : g_models) ctxs.push_back(gptoss_model_moe_ctx(m));
    for (gptoss_model *m : g_models)
      if (gptoss_comm_attach_local(gptoss_model_moe_ctx(m), ctxs.data())) die("cannot attach the GPUs to one another", m);
  }
}

long long inference(Transformer *transformer, Tokenizer *tokenizer, Sampler *sampler, Requests *requests) {
  (void)sampler;  // greedy, like the reference engine (argmax on the device)
  const Config &cfg = transformer->config;
  if (requests->max_seq_len > g_max_seq) {
    fprintf(stderr, "gptoss_b200: %d steps requested but the KV cache holds %d positions (GPTOSS_MAX_SEQ)\n",
            requests->max_seq_len, g_max_seq);
    exit(EXIT_FAILURE);
  }
  const int n_batches = (requests->num_reqs + g_batch - 1) / g_batch;
  std::atomic<int> next_batch{0};
  std::atomic<long long> total{0};
  std::vector<std::thread> workers;
  if (g_group) {  // one thread per rank; every batch is decoded by all of them together
    GroupSync sync((int)g_models.size());
    for (int r = 0; r < (int)g_models.size(); ++r)
      workers.emplace_back([&, r] {
        for (int b = 0; b < n_batches; ++b) {
          const int first = b * g_batch, n = std::min(g_batch, requests->num_reqs - first);
          total += run_batch(g_models[r], tokenizer, cfg, requests, first, n, &sync, r);
        }
      });
    for (auto &w : workers) w.join();
    return total;
  }
  if (g_continuous) {  // every replica refills its slots from one queue of requests
    std::atomic<int> next_req{0};
    for (gptoss_model *model : g_models)
      workers.emplace_back([&, model] { total += run_continuous(model, tokenizer, cfg, requests, next_req); });
    for (auto &w : workers) w.join();
    return total;
  }
  for (gptoss_model *model : g_models)
    workers.emplace_back([&, model] {
      for (int b = next_batch++; b < n_batches; b = next_batch++) {
        const int first = b * g_batch, n = std::min(g_batch, requests->num_reqs - first);
        total += run_batch(model, tokenizer, cfg, requests, first, n);
      }
    });
  for (auto &w : workers) w.join();
  return total;
}

void finish(Transformer *transformer, Tokenizer *tokenizer) {
  (void)transformer;
  (void)tokenizer;
  for (gptoss_model *m : g_models) gptoss_model_destroy(m);
  g_models.clear();
}

#endif  // GETP_RUN
