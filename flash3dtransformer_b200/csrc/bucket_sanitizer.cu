// Host-side scoreboard check of a finished PSH bucketing, the operator the reference binds as
// batch_bucket_sanitizer_cpu (src/psh/bucket_sanitizer_cpu.cpp:92-176, binding src/f3d_frontend.cu:133, call site
// tests/test_psh.py:127-129).  It runs on HOST copies of the buffers (the reference moves every tensor to the CPU
// first, :104-110) and has no kernel: every point takes one unit off its bucket's residual count and marks its
// (scene, bucket, offset) slot in an int8 table; afterwards every slot below a bucket's count must have been marked
// exactly once.  The residual and the table are written back in place, like the reference's copy_ at :172-173.
//
// The reference throws std::runtime_error with the position of the first violation; here the same text goes to
// f3d_last_error() and the status is F3D_ERR_ARG, which the Python operator turns into RuntimeError.
#include "f3d_common.cuh"
#include "../../include/f3d_b200.h"

extern "C" int f3d_batch_bucket_sanitizer_cpu(
    const void *bucket_id_, const void *bucket_counter_, const void *bucket_offset_, void *offset_check_table_,
    void *bucket_residual_, const void *batch_sep_, const void *offset_maxcnt_, uint32_t total_N,
    uint32_t batch_size, uint32_t num_bucket, uint32_t table_slots) {
  const uint16_t *bucket_id = (const uint16_t *)bucket_id_;
  const uint32_t *counter = (const uint32_t *)bucket_counter_;
  const uint32_t *offset = (const uint32_t *)bucket_offset_;
  int8_t *table = (int8_t *)offset_check_table_;
  uint32_t *residual = (uint32_t *)bucket_residual_;
  const uint32_t *sep = (const uint32_t *)batch_sep_;
  const uint32_t *maxcnt = (const uint32_t *)offset_maxcnt_;
  if (!bucket_id || !counter || !offset || !table || !residual || !sep || !maxcnt)
    return f3d::set_error(F3D_ERR_ARG, "batch_bucket_sanitizer_cpu: null buffer");
  if (batch_size && sep[batch_size - 1] > total_N)
    return f3d::set_error(F3D_ERR_ARG, "batch_bucket_sanitizer_cpu: batch_sep ends at %u but bucket_id holds %u points",
                          sep[batch_size - 1], total_N);
  // marking pass
  for (uint32_t bid = 0; bid < batch_size; ++bid) {
    const uint32_t begin = bid ? sep[bid - 1] : 0u, end = sep[bid];
    for (uint32_t c = begin; c < end; ++c) {
      const uint32_t id = bucket_id[c], off = offset[c];
      if (id >= num_bucket || off >= maxcnt[bid] || off >= table_slots)
        return f3d::set_error(F3D_ERR_ARG, "col=%u: buckid=%u|num_bucket=%u, buckoff=%u|offset_maxcnt=%u, overflow ",
                              c, id, num_bucket, off, maxcnt[bid]);
      residual[(size_t)bid * num_bucket + id] -= 1u;
      table[((size_t)bid * num_bucket + id) * table_slots + off] += 1;
    }
  }
  // every slot below a bucket's count holds exactly one point
  for (uint32_t bid = 0; bid < batch_size; ++bid)
    for (uint32_t b = 0; b < num_bucket; ++b) {
      const uint32_t cnt = counter[(size_t)bid * num_bucket + b];
      if (cnt > table_slots)
        return f3d::set_error(F3D_ERR_ARG, "batchid=%u buck=%u: count %u exceeds the table's %u slots", bid, b, cnt,
                              table_slots);
      const int8_t *row = table + ((size_t)bid * num_bucket + b) * table_slots;
      for (uint32_t s = 0; s < cnt; ++s)
        if (row[s] != 1)
          return f3d::set_error(F3D_ERR_ARG, "Wrong scoreboard, batchid=%u buck=%u,[Slot=%u|MaxCnt=%u],Score=%d", bid, b,
                                s, cnt, (int)row[s]);
    }
  return F3D_OK;
}
