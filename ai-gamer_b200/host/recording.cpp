// recording.cpp -- reader for the recording files the reference's input recorder writes, and batched offline
// inference over them.
//
// File layout (little endian, no padding; input_recorder.cpp:24-27 writes the header, :122-133 every record):
//   int32 width, int32 height
//   per frame:  uint16 keyStates, int32 mouseDeltaX, int32 mouseDeltaY        (10 bytes)
//               uint8 planar RGB frame: plane R, plane G, plane B, width*height bytes each
// Records are indexed the way ReadStateData does (main.cpp:41-92): only whole records count, a partial one at
// the end of the file is ignored.  Targets follow Train.cpp:70-76: button j = bit j of keyStates (14 buttons),
// axes = mouse deltas / 256.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>

#include "aig_b200.h"
#include "aig_host.h"

struct aig_recording {
  FILE* f = nullptr;
  int width = 0, height = 0;
  long long n_records = 0;
  size_t frame_bytes = 0, stride = 0;
  std::string err;
};

namespace {
constexpr long long kHeaderBytes = 8, kRecordHeader = 10;
std::string g_open_error;
int rfail(aig_recording* r, int code, const std::string& msg) {
  r->err = msg;
  return code;
}
}  // namespace

extern "C" {

const char* aig_recording_last_error(aig_recording* r) { return r ? r->err.c_str() : g_open_error.c_str(); }

int aig_recording_open(const char* path, aig_recording** out) {
  if (!path || !out) return AIG_ERR_INVALID;
  *out = nullptr;
  FILE* f = fopen(path, "rb");
  if (!f) {
    g_open_error = std::string("cannot open ") + path;
    return AIG_ERR_IO;
  }
  int32_t wh[2] = {0, 0};
  if (fread(wh, 4, 2, f) != 2 || wh[0] <= 0 || wh[1] <= 0 || (long long)wh[0] * wh[1] > (1ll << 28)) {
    fclose(f);
    g_open_error = std::string("no valid width/height header in ") + path;
    return AIG_ERR_IO;
  }
  aig_recording* r = new aig_recording();
  r->f = f;
  r->width = wh[0];
  r->height = wh[1];
  r->frame_bytes = (size_t)3 * wh[0] * wh[1];
  r->stride = (size_t)kRecordHeader + r->frame_bytes;
  fseeko(f, 0, SEEK_END);
  const long long size = (long long)ftello(f);
  r->n_records = (size - kHeaderBytes) / (long long)r->stride;  // whole records only
  *out = r;
  return AIG_OK;
}

int aig_recording_close(aig_recording* r) {
  if (!r) return AIG_OK;
  if (r->f) fclose(r->f);
  delete r;
  return AIG_OK;
}

int aig_recording_info(const aig_recording* r, int* width, int* height, long long* n_records) {
  if (!r) return AIG_ERR_INVALID;
  if (width) *width = r->width;
  if (height) *height = r->height;
  if (n_records) *n_records = r->n_records;
  return AIG_OK;
}

// `count` consecutive records from `first`: frames [count][3][height][width] as stored, key_states [count],
// mouse_dxdy [count][2]; any of the three may be null
int aig_recording_read(aig_recording* r, long long first, int count, uint8_t* frames, uint16_t* key_states, int32_t* mouse_dxdy) {
  if (!r || count < 0) return AIG_ERR_INVALID;
  if (first < 0 || first + count > r->n_records) return rfail(r, AIG_ERR_INVALID, "record range outside the file");
  for (int i = 0; i < count; ++i) {
    if (fseeko(r->f, (off_t)(kHeaderBytes + (first + i) * (long long)r->stride), SEEK_SET) != 0) return rfail(r, AIG_ERR_IO, "seek failed");
    unsigned char hdr[kRecordHeader];
    if (fread(hdr, 1, kRecordHeader, r->f) != (size_t)kRecordHeader) return rfail(r, AIG_ERR_IO, "short read of a record header");
    if (key_states) memcpy(&key_states[i], hdr, 2);
    if (mouse_dxdy) {
      memcpy(&mouse_dxdy[2 * i], hdr + 2, 4);
      memcpy(&mouse_dxdy[2 * i + 1], hdr + 6, 4);
    }
    if (frames && fread(frames + (size_t)i * r->frame_bytes, 1, r->frame_bytes, r->f) != r->frame_bytes)
      return rfail(r, AIG_ERR_IO, "short read of a frame");
  }
  return AIG_OK;
}

// Train.cpp:70-76: targets [count][16]
int aig_recording_targets(const uint16_t* key_states, const int32_t* mouse_dxdy, int count, float* targets) {
  if (!key_states || !mouse_dxdy || !targets || count < 0) return AIG_ERR_INVALID;
  for (int i = 0; i < count; ++i) {
    for (int j = 0; j < 14; ++j) targets[i * 16 + j] = (float)((key_states[i] >> j) & 1);
    targets[i * 16 + 14] = (float)mouse_dxdy[2 * i] / 256.0f;
    targets[i * 16 + 15] = (float)mouse_dxdy[2 * i + 1] / 256.0f;
  }
  return AIG_OK;
}

// Offline inference over records [first, first + count): batches of the encoder's batch size go through the
// pipelined host entry point as planar RGB (the bytes of the file, untouched); the last batch is padded by
// repeating its final frame.  out_host [count][n_out] fp32 (host memory).  n_out is the encoder's.
int aig_cnn_infer_recording(aig_cnn* m, aig_recording* r, long long first, long long count, int batch, int n_out, float* out_host) {
  if (!m || !r || !out_host || batch <= 0 || n_out <= 0 || count < 0) return AIG_ERR_INVALID;
  if (first < 0 || first + count > r->n_records) return rfail(r, AIG_ERR_INVALID, "record range outside the file");
  uint8_t* stage[2] = {nullptr, nullptr};
  float* outs[2] = {nullptr, nullptr};
  const size_t fb = (size_t)batch * r->frame_bytes, ob = (size_t)batch * n_out * sizeof(float);
  int rc = AIG_OK;
  for (int s = 0; s < 2 && rc == AIG_OK; ++s)
    if (cudaMallocHost(reinterpret_cast<void**>(&stage[s]), fb) != cudaSuccess || cudaMallocHost(reinterpret_cast<void**>(&outs[s]), ob) != cudaSuccess)
      rc = rfail(r, AIG_ERR_CUDA, "pinned staging allocation failed");
  const long long n_batches = (count + batch - 1) / batch;
  auto collect = [&](long long b) {
    const int s = (int)(b & 1);
    int w = aig_cnn_wait(m, s);
    if (w != AIG_OK) return w;
    const long long lo = b * batch, n = (count - lo < batch) ? count - lo : batch;
    memcpy(out_host + (size_t)lo * n_out, outs[s], (size_t)n * n_out * sizeof(float));
    return (int)AIG_OK;
  };
  for (long long b = 0; b < n_batches && rc == AIG_OK; ++b) {
    const int s = (int)(b & 1);
    if (b >= 2) rc = collect(b - 2);
    if (rc != AIG_OK) break;
    const long long lo = b * batch;
    const int n = (int)((count - lo < batch) ? count - lo : batch);
    rc = aig_recording_read(r, first + lo, n, stage[s], nullptr, nullptr);
    for (int i = n; i < batch && rc == AIG_OK; ++i) memcpy(stage[s] + (size_t)i * r->frame_bytes, stage[s] + (size_t)(n - 1) * r->frame_bytes, r->frame_bytes);
    if (rc == AIG_OK) rc = aig_cnn_submit_host_rgb(m, s, stage[s], outs[s]);
    if (rc != AIG_OK && r->err.empty()) rfail(r, rc, aig_cnn_last_error(m));
  }
  for (long long b = (n_batches >= 2 ? n_batches - 2 : 0); b < n_batches && rc == AIG_OK; ++b) rc = collect(b);
  for (int s = 0; s < 2; ++s) {
    cudaFreeHost(stage[s]);
    cudaFreeHost(outs[s]);
  }
  return rc;
}

}  // extern "C"
