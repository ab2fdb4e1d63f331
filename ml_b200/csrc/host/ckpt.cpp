// Checkpoint IO.
//
// Layout (csrc/src/checkpoint.cu:44-118, csrc/include/checkpoint.h:14-19 in the reference):
//   <dir>/step_<N>/meta.bin              raw struct {int64 step; float loss; int64 tokens_seen; int version}
//                                        (32 bytes with natural x86-64 padding, version = 1)
//   <dir>/step_<N>/weights_rank_<r>.bin  this rank's contiguous shard of the flat fp32 master buffer
// The reference forms the weight path but never writes the payload; here it is written, together with
//   optim_rank_<r>.bin (m then v of the same shard), vision_rank_<r>.bin, state_rank_<r>.bin
// by a background IO thread from a host snapshot, each file published atomically (write "<name>.tmp",
// fsync, rename) so a reader never sees a torn file.
#include <cerrno>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <fcntl.h>
#include <mutex>
#include <string>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>

namespace {

struct Meta {
  int64_t step;
  float loss;
  int64_t tokens_seen;
  int32_t version;
};
static_assert(sizeof(Meta) == 32, "meta.bin must be 32 bytes");

int write_atomic(const std::string& path, const void* p, size_t n) {
  std::string tmp = path + ".tmp";
  int fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) return errno ? errno : 1;
  const char* c = (const char*)p;
  size_t left = n;
  while (left) {
    ssize_t w = write(fd, c, left > (1u << 30) ? (1u << 30) : left);
    if (w < 0) { if (errno == EINTR) continue; int e = errno; close(fd); return e ? e : 1; }
    c += w; left -= (size_t)w;
  }
  fsync(fd);
  close(fd);
  if (rename(tmp.c_str(), path.c_str()) != 0) return errno ? errno : 1;
  return 0;
}

struct Job { std::string path; const void* p; size_t n; };
struct Writer {
  std::thread th;
  std::mutex mu;
  std::condition_variable cv, cv_idle;
  std::deque<Job> q;
  int inflight = 0, first_err = 0;
  bool stop = false;
};

void run(Writer* w) {
  for (;;) {
    Job j;
    {
      std::unique_lock<std::mutex> lk(w->mu);
      w->cv.wait(lk, [&] { return w->stop || !w->q.empty(); });
      if (w->q.empty()) return;
      j = w->q.front();
      w->q.pop_front();
    }
    int e = write_atomic(j.path, j.p, j.n);
    {
      std::lock_guard<std::mutex> lk(w->mu);
      if (e && !w->first_err) w->first_err = e;
      w->inflight--;
    }
    w->cv_idle.notify_all();
  }
}

}  // namespace

extern "C" {

int mlb_mkdirs(const char* path) {
  std::string s(path);
  for (size_t i = 1; i <= s.size(); i++) {
    if (i == s.size() || s[i] == '/') {
      std::string sub = s.substr(0, i);
      if (mkdir(sub.c_str(), 0755) != 0 && errno != EEXIST) return errno;
    }
  }
  return 0;
}

int mlb_ckpt_write_meta(const char* step_dir, int64_t step, float loss, int64_t tokens_seen) {
  Meta m;
  memset(&m, 0, sizeof m);
  m.step = step; m.loss = loss; m.tokens_seen = tokens_seen; m.version = 1;
  return write_atomic(std::string(step_dir) + "/meta.bin", &m, sizeof m);
}

// Returns 0 on success, 1 if missing (caller starts fresh), 2 if short/corrupt or wrong version.
int mlb_ckpt_read_meta(const char* step_dir, int64_t* step, float* loss, int64_t* tokens_seen) {
  std::string p = std::string(step_dir) + "/meta.bin";
  FILE* f = fopen(p.c_str(), "rb");
  if (!f) return 1;
  Meta m;
  size_t r = fread(&m, 1, sizeof m, f);
  fclose(f);
  if (r != sizeof m || m.version != 1) return 2;
  *step = m.step; *loss = m.loss; *tokens_seen = m.tokens_seen;
  return 0;
}

int mlb_write_blob(const char* path, const void* p, int64_t nbytes) { return write_atomic(path, p, (size_t)nbytes); }

// Returns 0 ok, 1 missing, 2 size mismatch (truncated file), 3 read error.
int mlb_read_blob(const char* path, void* p, int64_t nbytes) {
  struct stat st;
  if (stat(path, &st) != 0) return 1;
  if ((int64_t)st.st_size != nbytes) return 2;
  FILE* f = fopen(path, "rb");
  if (!f) return 1;
  size_t r = fread(p, 1, (size_t)nbytes, f);
  fclose(f);
  return r == (size_t)nbytes ? 0 : 3;
}

void* mlb_writer_create() {
  Writer* w = new Writer;
  w->th = std::thread(run, w);
  return w;
}
// The memory must stay valid until mlb_writer_wait returns.
void mlb_writer_submit(void* h, const char* path, const void* p, int64_t nbytes) {
  Writer* w = (Writer*)h;
  {
    std::lock_guard<std::mutex> lk(w->mu);
    w->q.push_back({path, p, (size_t)nbytes});
    w->inflight++;
  }
  w->cv.notify_one();
}
int mlb_writer_wait(void* h) {
  Writer* w = (Writer*)h;
  std::unique_lock<std::mutex> lk(w->mu);
  w->cv_idle.wait(lk, [&] { return w->inflight == 0; });
  int e = w->first_err;
  w->first_err = 0;
  return e;
}
void mlb_writer_destroy(void* h) {
  Writer* w = (Writer*)h;
  if (!w) return;
  {
    std::lock_guard<std::mutex> lk(w->mu);
    w->stop = true;
  }
  w->cv.notify_all();
  w->th.join();
  delete w;
}

}  // extern "C"
