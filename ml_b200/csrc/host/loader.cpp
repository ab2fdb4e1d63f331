// Token loader core + prefetching batch pipe.
//
// File format (llm.c ".bin"): 64 x int32 header, header[0] == 20240520, header[2] == token count,
// then uint16 tokens.  A batch is a window of B*T+1 tokens at `pos`: ids[i] = w[i], tgt[i] = w[i+1];
// pos advances by B*T and wraps to 0 when the next window would overrun the file
// (semantics of train/gpt.cu:925-945).  Unlike the reference (fseek+fread on the training thread) the
// file is mmap'ed and windows are expanded to int32 by a worker thread directly into caller-provided
// (pinned) slots, so the training thread never touches the disk.
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <fcntl.h>
#include <mutex>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace {

// One mapped token file.  `base` = tokens in the shards before it: a position handed to the caller is base + offset.
struct Shard {
  int fd = -1;
  const uint8_t* map = nullptr;
  size_t map_bytes = 0;
  const uint16_t* tok = nullptr;
  int64_t ntok = 0, base = 0;
};

struct Loader {
  // A data set is one file or several shards read one after the other (a window never spans two shards; the tail of a
  // shard that does not hold a whole window is skipped, as at the end of a single file).  tok / ntok / pos describe the
  // shard being read.
  std::vector<Shard> shards;
  int cur = 0;
  const uint16_t* tok = nullptr;
  int64_t ntok = 0, pos = 0;
  int B = 0, T = 0;
  // Data-parallel striping: this reader serves windows `first`, `first + every`, `first + 2*every`, ... of the file (a
  // window is B*T tokens), so `every` ranks with first = 0..every-1 read disjoint windows, prefetch included.
  int64_t first = 0, every = 1;
  // Vocabulary check (0 = off): the first window holding a token >= vocab is remembered; the reader of that window
  // asks with mlb_loader_bad() before the tokens reach the device (the kernels index tables by token id).
  int vocab = 0;
  std::atomic<int64_t> bad_pos{-1};
  std::atomic<int> bad_tok{0};
};

struct Job { int slot; int32_t* ids; int32_t* tgt; };

struct Pipe {
  Loader* ld;
  std::thread th;
  std::mutex mu;
  std::condition_variable cv_job, cv_done;
  std::deque<Job> jobs;
  std::vector<int> done;  // per-slot completion counters
  std::vector<int> want;
  std::vector<int64_t> slot_pos;
  bool stop = false;
};

void fill(Loader* ld, int32_t* ids, int32_t* tgt) {
  const int64_t n = (int64_t)ld->B * ld->T;
  if (ld->pos + n + 1 > ld->ntok) {
    // on to the next shard (the only one, again, for a single file), at this reader's first window
    ld->cur = (ld->cur + 1) % (int)ld->shards.size();
    ld->tok = ld->shards[ld->cur].tok;
    ld->ntok = ld->shards[ld->cur].ntok;
    ld->pos = ld->first * n;
  }
  const uint16_t* w = ld->tok + ld->pos;
  uint16_t mx = w[0];
  for (int64_t i = 0; i < n; i++) { ids[i] = w[i]; tgt[i] = w[i + 1]; mx = w[i + 1] > mx ? w[i + 1] : mx; }
  if (ld->vocab > 0 && (int)mx >= ld->vocab && ld->bad_pos.load() < 0) {
    ld->bad_tok.store(mx);
    ld->bad_pos.store(ld->shards[ld->cur].base + ld->pos);
  }
  ld->pos += n * ld->every;
}

void worker(Pipe* p) {
  for (;;) {
    Job j;
    {
      std::unique_lock<std::mutex> lk(p->mu);
      p->cv_job.wait(lk, [&] { return p->stop || !p->jobs.empty(); });
      if (p->stop && p->jobs.empty()) return;
      j = p->jobs.front();
      p->jobs.pop_front();
    }
    int64_t before = p->ld->pos;
    fill(p->ld, j.ids, j.tgt);
    {
      std::lock_guard<std::mutex> lk(p->mu);
      p->slot_pos[j.slot] = before;
      p->done[j.slot]++;
    }
    p->cv_done.notify_all();
  }
}

}  // namespace

extern "C" {

// Maps one token file; 0 or the error code of mlb_loader_open.  `need` = tokens a shard must hold at least.
static int map_shard(const char* path, int64_t need, Shard* out) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) return 1;
  struct stat st;
  if (fstat(fd, &st) != 0 || (size_t)st.st_size < 256) { close(fd); return 2; }
  void* m = mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  if (m == MAP_FAILED) { close(fd); return 1; }
  const int32_t* h = (const int32_t*)m;
  if (h[0] != 20240520) { munmap(m, st.st_size); close(fd); return 2; }
  int64_t ntok = h[2];
  int64_t have = ((int64_t)st.st_size - 256) / 2;
  if (ntok <= 0 || ntok > have) ntok = have;  // truncated file, or a count that does not fit the header's int32: serve what is there
  if (ntok < need) { munmap(m, st.st_size); close(fd); return 3; }
  madvise(m, st.st_size, MADV_SEQUENTIAL);
  out->fd = fd; out->map = (const uint8_t*)m; out->map_bytes = st.st_size;
  out->tok = (const uint16_t*)((const uint8_t*)m + 256);
  out->ntok = ntok;
  return 0;
}

// Returns a handle or nullptr; *err: 1 = cannot open, 2 = bad magic / short header, 3 = too few tokens.
void* mlb_loader_open(const char* path, int B, int T, int* err) {
  Shard sh;
  *err = map_shard(path, (int64_t)B * T + 1, &sh);
  if (*err) return nullptr;
  Loader* ld = new Loader;
  ld->shards.push_back(sh);
  ld->tok = sh.tok; ld->ntok = sh.ntok; ld->B = B; ld->T = T;
  return ld;
}
// Appends another shard of the same data set (read after the ones before it); same error codes, 0 = ok.  Call before
// the first window is read.
int mlb_loader_add(void* h, const char* path) {
  Loader* ld = (Loader*)h;
  Shard sh;
  int err = map_shard(path, (int64_t)ld->B * ld->T + 1, &sh);
  if (err) return err;
  sh.base = ld->shards.back().base + ld->shards.back().ntok;
  ld->shards.push_back(sh);
  return 0;
}
int64_t mlb_loader_ntok(void* h) {
  Loader* ld = (Loader*)h;
  return ld->shards.back().base + ld->shards.back().ntok;
}
int64_t mlb_loader_pos(void* h) {
  Loader* ld = (Loader*)h;
  return ld->shards[ld->cur].base + ld->pos;
}
void mlb_loader_set_pos(void* h, int64_t pos) {
  Loader* ld = (Loader*)h;
  int c = 0;
  while (c + 1 < (int)ld->shards.size() && pos >= ld->shards[c + 1].base) c++;
  ld->cur = c;
  ld->tok = ld->shards[c].tok;
  ld->ntok = ld->shards[c].ntok;
  ld->pos = pos - ld->shards[c].base;
}
// Reader `first` of `every` (data-parallel rank / world).  Returns 1 if the file is too short for that many disjoint
// readers (fewer than `every` whole windows), else 0; the position moves to the reader's first window.
int mlb_loader_set_stride(void* h, int64_t first, int64_t every) {
  Loader* ld = (Loader*)h;
  const int64_t n = (int64_t)ld->B * ld->T;
  if (every < 1 || first < 0 || first >= every) return 1;
  for (const Shard& sh : ld->shards)
    if (every * n + 1 > sh.ntok) return 1;      // every shard must hold a window for every reader
  ld->first = first; ld->every = every;
  ld->cur = 0; ld->tok = ld->shards[0].tok; ld->ntok = ld->shards[0].ntok; ld->pos = first * n;
  return 0;
}
void mlb_loader_next(void* h, int32_t* ids, int32_t* tgt) { fill((Loader*)h, ids, tgt); }
// Tokens >= vocab are reported from now on (vocab 0 switches the check off).
void mlb_loader_set_vocab(void* h, int vocab) { ((Loader*)h)->vocab = vocab; }
// 1 if a window with a token >= vocab has been served: *pos = its file position, *tok = its largest token.
int mlb_loader_bad(void* h, int64_t* pos, int* tok) {
  Loader* ld = (Loader*)h;
  const int64_t p = ld->bad_pos.load();
  if (p < 0) return 0;
  *pos = p; *tok = ld->bad_tok.load();
  return 1;
}
void mlb_loader_close(void* h) {
  Loader* ld = (Loader*)h;
  if (!ld) return;
  for (const Shard& sh : ld->shards) {
    munmap((void*)sh.map, sh.map_bytes);
    close(sh.fd);
  }
  delete ld;
}

void* mlb_pipe_create(void* loader, int nslots) {
  Pipe* p = new Pipe;
  p->ld = (Loader*)loader;
  p->done.assign(nslots, 0);
  p->want.assign(nslots, 0);
  p->slot_pos.assign(nslots, 0);
  p->th = std::thread(worker, p);
  return p;
}
// Queue an asynchronous refill of `slot` (windows are served in submission order).
void mlb_pipe_submit(void* h, int slot, int32_t* ids, int32_t* tgt) {
  Pipe* p = (Pipe*)h;
  {
    std::lock_guard<std::mutex> lk(p->mu);
    p->want[slot]++;
    p->jobs.push_back({slot, ids, tgt});
  }
  p->cv_job.notify_one();
}
// Block until every refill submitted for `slot` has finished; returns the file position it was cut from.
int64_t mlb_pipe_wait(void* h, int slot) {
  Pipe* p = (Pipe*)h;
  std::unique_lock<std::mutex> lk(p->mu);
  p->cv_done.wait(lk, [&] { return p->done[slot] >= p->want[slot]; });
  return p->slot_pos[slot];
}
void mlb_pipe_destroy(void* h) {
  Pipe* p = (Pipe*)h;
  if (!p) return;
  {
    std::lock_guard<std::mutex> lk(p->mu);
    p->stop = true;
  }
  p->cv_job.notify_all();
  p->th.join();
  delete p;
}

// Writes a .bin file in the same format (used by tests and synthetic-shard generation).
int mlb_write_token_bin(const char* path, const uint16_t* tok, int64_t n) {
  FILE* f = fopen(path, "wb");
  if (!f) return 1;
  int32_t h[64];
  memset(h, 0, sizeof h);
  h[0] = 20240520; h[1] = 1; h[2] = (int32_t)n;
  int bad = fwrite(h, 4, 64, f) != 64 || fwrite(tok, 2, n, f) != (size_t)n;
  fclose(f);
  return bad ? 2 : 0;
}

}  // extern "C"
