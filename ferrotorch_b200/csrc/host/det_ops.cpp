// Detection operators on the host: greedy non-maximum suppression and RoI align over fp32 data
// (the reference keeps them native too: ferrotorch-vision/src/ops.rs:209 ``nms``, :751 ``roi_align``).
//
//   ftd_nms        boxes [n, 4] (x1, y1, x2, y2) already sorted by score, highest first; writes
//                  the positions of the kept boxes in that order and returns their number.  A box
//                  is dropped when its IoU with a kept box is ABOVE the threshold.  The sweep keeps
//                  one bit per box and only compares a candidate with the boxes kept so far.
//   ftd_roi_align  feat [N, C, H, W], rois [K, 5] (batch index, x1, y1, x2, y2) -> out [K, C, ph, pw];
//                  each output bin is the mean of sampling^2 bilinear samples; a sample more than
//                  one pixel outside the map contributes 0, coordinates are clamped to the map.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

#define FTD_API extern "C" __attribute__((visibility("default")))

FTD_API long long ftd_nms(const float* boxes, long long n, float iou_threshold, long long* keep) {
  if (!boxes || !keep || n < 0) return -1;
  std::vector<float> area(static_cast<size_t>(n));
  for (long long i = 0; i < n; ++i) {
    const float* b = boxes + 4 * i;
    area[i] = (b[2] - b[0]) * (b[3] - b[1]);
  }
  long long kept = 0;
  for (long long i = 0; i < n; ++i) {
    const float* a = boxes + 4 * i;
    bool drop = false;
    for (long long t = 0; t < kept && !drop; ++t) {
      const long long j = keep[t];
      const float* b = boxes + 4 * j;
      const float w = std::min(a[2], b[2]) - std::max(a[0], b[0]);
      const float h = std::min(a[3], b[3]) - std::max(a[1], b[1]);
      if (w <= 0.f || h <= 0.f) continue;
      const float inter = w * h;
      drop = inter / (area[i] + area[j] - inter) > iou_threshold;
    }
    if (!drop) keep[kept++] = i;
  }
  return kept;
}

namespace {

struct Tap {
  int p00, p01, p10, p11;
  float w00, w01, w10, w11;
};

inline Tap make_tap(float y, float x, int H, int W) {
  Tap t{0, 0, 0, 0, 0.f, 0.f, 0.f, 0.f};
  if (y < -1.f || y > static_cast<float>(H) || x < -1.f || x > static_cast<float>(W)) return t;
  y = std::max(y, 0.f);
  x = std::max(x, 0.f);
  int y0 = static_cast<int>(y), x0 = static_cast<int>(x), y1, x1;
  if (y0 >= H - 1) { y0 = y1 = H - 1; y = static_cast<float>(y0); } else { y1 = y0 + 1; }
  if (x0 >= W - 1) { x0 = x1 = W - 1; x = static_cast<float>(x0); } else { x1 = x0 + 1; }
  const float ly = y - y0, lx = x - x0, hy = 1.f - ly, hx = 1.f - lx;
  t.p00 = y0 * W + x0; t.p01 = y0 * W + x1; t.p10 = y1 * W + x0; t.p11 = y1 * W + x1;
  t.w00 = hy * hx; t.w01 = hy * lx; t.w10 = ly * hx; t.w11 = ly * lx;
  return t;
}

}  // namespace

FTD_API int ftd_roi_align(const float* feat, int N, int C, int H, int W, const float* rois, long long K, int ph, int pw,
                          float spatial_scale, int sampling, int aligned, float* out) {
  if (!feat || !rois || !out || N <= 0 || C <= 0 || H <= 0 || W <= 0 || K < 0 || ph <= 0 || pw <= 0 || sampling <= 0) return -1;
  const float off = aligned ? 0.5f : 0.f;
  std::vector<Tap> taps(static_cast<size_t>(ph) * pw * sampling * sampling);
  for (long long k = 0; k < K; ++k) {
    const float* r = rois + 5 * k;
    const int b = static_cast<int>(r[0]);
    if (b < 0 || b >= N) return -2;
    const float x1 = r[1] * spatial_scale - off, y1 = r[2] * spatial_scale - off;
    float rw = r[3] * spatial_scale - off - x1, rh = r[4] * spatial_scale - off - y1;
    if (!aligned) { rw = std::max(rw, 1.f); rh = std::max(rh, 1.f); }
    const float bw = rw / pw, bh = rh / ph;
    size_t t = 0;
    for (int py = 0; py < ph; ++py)
      for (int px = 0; px < pw; ++px)
        for (int iy = 0; iy < sampling; ++iy)
          for (int ix = 0; ix < sampling; ++ix)
            taps[t++] = make_tap(y1 + py * bh + (iy + 0.5f) * bh / sampling, x1 + px * bw + (ix + 0.5f) * bw / sampling, H, W);
    const float inv = 1.f / (sampling * sampling);
    for (int c = 0; c < C; ++c) {
      const float* f = feat + (static_cast<size_t>(b) * C + c) * H * W;
      float* o = out + (static_cast<size_t>(k) * C + c) * ph * pw;
      t = 0;
      for (int bin = 0; bin < ph * pw; ++bin) {
        float acc = 0.f;
        for (int s = 0; s < sampling * sampling; ++s, ++t) {
          const Tap& q = taps[t];
          acc += q.w00 * f[q.p00] + q.w01 * f[q.p01] + q.w10 * f[q.p10] + q.w11 * f[q.p11];
        }
        o[bin] = acc * inv;
      }
    }
  }
  return 0;
}
