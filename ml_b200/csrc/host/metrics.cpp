// Metrics writers: one JSON line per log call plus a TensorBoard event file.
//
// JSONL keys and TensorBoard tags follow the reference's logger (csrc/src/metrics.cu:187-200):
//   {"step","wall_time","loss","lr","tokens_seen","step_time_ms","cuda_mem_free","cuda_mem_total"}
//   train/loss, train/lr, train/tokens_seen, train/step_time_ms, cuda/mem_free, cuda/mem_total
// plus any number of extra named scalars (device-timed step, exposed-communication ms, MFU ...).
// TFEvents framing: [u64 len][u32 masked crc32c(len)][payload][u32 masked crc32c(payload)], payload =
// protobuf Event{1: wall_time double, 2: step int64, 3: file_version string | 5: Summary{1: Value{1: tag, 2: simple_value}}}.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <string>
#include <sys/time.h>
#include <unistd.h>

namespace {

uint32_t crc_table[256];
bool crc_init_done = false;
void crc_init() {
  for (uint32_t i = 0; i < 256; i++) {
    uint32_t c = i;
    for (int k = 0; k < 8; k++) c = (c & 1) ? (c >> 1) ^ 0x82F63B78u : c >> 1;
    crc_table[i] = c;
  }
  crc_init_done = true;
}
uint32_t crc32c(const void* p, size_t n) {
  if (!crc_init_done) crc_init();
  uint32_t c = 0xFFFFFFFFu;
  const uint8_t* b = (const uint8_t*)p;
  for (size_t i = 0; i < n; i++) c = crc_table[(c ^ b[i]) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}
uint32_t masked(uint32_t crc) { return ((crc >> 15) | (crc << 17)) + 0xa282ead8u; }

void put_varint(std::string& s, uint64_t v) {
  while (v >= 0x80) { s.push_back((char)(v | 0x80)); v >>= 7; }
  s.push_back((char)v);
}
void put_bytes(std::string& s, int field, const std::string& b) {
  put_varint(s, (uint64_t)(field << 3 | 2));
  put_varint(s, b.size());
  s += b;
}

double now_s() {
  struct timeval tv;
  gettimeofday(&tv, nullptr);
  return tv.tv_sec + tv.tv_usec * 1e-6;
}

struct Metrics {
  FILE* jsonl = nullptr;
  FILE* tb = nullptr;
};

void write_record(FILE* f, const std::string& payload) {
  uint64_t len = payload.size();
  uint32_t c1 = masked(crc32c(&len, 8)), c2 = masked(crc32c(payload.data(), payload.size()));
  fwrite(&len, 8, 1, f); fwrite(&c1, 4, 1, f);
  fwrite(payload.data(), 1, payload.size(), f); fwrite(&c2, 4, 1, f);
}

std::string event_header(double wall, int64_t step) {
  std::string e;
  e.push_back(0x09);
  e.append((const char*)&wall, 8);
  e.push_back(0x10);
  put_varint(e, (uint64_t)step);
  return e;
}

void tb_scalar(FILE* f, double wall, int64_t step, const char* tag, float value) {
  std::string val;
  put_bytes(val, 1, tag);
  val.push_back(0x15);
  val.append((const char*)&value, 4);
  std::string summary;
  put_bytes(summary, 1, val);
  std::string e = event_header(wall, step);
  put_bytes(e, 5, summary);
  write_record(f, e);
}

}  // namespace

extern "C" {

uint32_t mlb_crc32c(const void* p, int64_t n) { return crc32c(p, (size_t)n); }

void* mlb_metrics_open(const char* dir, int tensorboard) {
  Metrics* m = new Metrics;
  std::string d(dir);
  m->jsonl = fopen((d + "/metrics.jsonl").c_str(), "a");
  if (!m->jsonl) { delete m; return nullptr; }
  if (tensorboard) {
    char host[128] = "host";
    gethostname(host, sizeof host - 1);
    char name[512];
    snprintf(name, sizeof name, "%s/events.out.tfevents.%ld.%s", dir, (long)time(nullptr), host);
    m->tb = fopen(name, "wb");
    if (m->tb) {
      std::string e = event_header(now_s(), 0);
      put_bytes(e, 3, "brain.Event:2");
      write_record(m->tb, e);
      fflush(m->tb);
    }
  }
  return m;
}

// extra_names / extra_vals: n_extra additional scalars, written to both sinks (TB tag "train/<name>").
void mlb_metrics_log(void* h, int64_t step, double loss, double lr, int64_t tokens_seen, double step_time_ms,
                     int64_t mem_free, int64_t mem_total, int n_extra, const char** extra_names,
                     const double* extra_vals) {
  Metrics* m = (Metrics*)h;
  double wall = now_s();
  fprintf(m->jsonl,
          "{\"step\":%lld,\"wall_time\":%.6f,\"loss\":%.6f,\"lr\":%.8g,\"tokens_seen\":%lld,"
          "\"step_time_ms\":%.4f,\"cuda_mem_free\":%lld,\"cuda_mem_total\":%lld",
          (long long)step, wall, loss, lr, (long long)tokens_seen, step_time_ms, (long long)mem_free,
          (long long)mem_total);
  for (int i = 0; i < n_extra; i++) fprintf(m->jsonl, ",\"%s\":%.8g", extra_names[i], extra_vals[i]);
  fprintf(m->jsonl, "}\n");
  fflush(m->jsonl);
  if (m->tb) {
    tb_scalar(m->tb, wall, step, "train/loss", (float)loss);
    tb_scalar(m->tb, wall, step, "train/lr", (float)lr);
    tb_scalar(m->tb, wall, step, "train/tokens_seen", (float)tokens_seen);
    tb_scalar(m->tb, wall, step, "train/step_time_ms", (float)step_time_ms);
    tb_scalar(m->tb, wall, step, "cuda/mem_free", (float)mem_free);
    tb_scalar(m->tb, wall, step, "cuda/mem_total", (float)mem_total);
    for (int i = 0; i < n_extra; i++) {
      std::string tag = std::string("train/") + extra_names[i];
      tb_scalar(m->tb, wall, step, tag.c_str(), (float)extra_vals[i]);
    }
    fflush(m->tb);
  }
}

// One scalar under its own tag (e.g. "eval/loss"): a JSONL line {"step", "wall_time", "<tag>"} and a TensorBoard event.
void mlb_metrics_scalar(void* h, int64_t step, const char* tag, double value) {
  Metrics* m = (Metrics*)h;
  if (!m) return;
  double wall = now_s();
  fprintf(m->jsonl, "{\"step\":%lld,\"wall_time\":%.6f,\"%s\":%.8g}\n", (long long)step, wall, tag, value);
  fflush(m->jsonl);
  if (m->tb) {
    tb_scalar(m->tb, wall, step, tag, (float)value);
    fflush(m->tb);
  }
}

void mlb_metrics_close(void* h) {
  Metrics* m = (Metrics*)h;
  if (!m) return;
  if (m->jsonl) fclose(m->jsonl);
  if (m->tb) fclose(m->tb);
  delete m;
}

}  // extern "C"
