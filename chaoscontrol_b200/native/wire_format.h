// Packed wire records of the episodic-memory control plane.
//
// These structs are a binary protocol: GPU ranks, the CPU controller process
// and the teacher rank exchange them through shared-memory rings, so field
// order, widths and total sizes are fixed (they match the reference's records
// byte for byte: kernels/_cpu_ssm_controller/src/wire_events.h:66-284).  Every
// size is pinned by a static_assert and exported through ccb_wire_sizeof() so
// the Python side can check its own mirror of the layout.
#pragma once
#include <cstddef>
#include <cstdint>

namespace ccb::wire {

constexpr int kKeyRepDim = 256;          // fp16 key / query representation
constexpr int kSpanLength = 4;           // value span (token ids)
constexpr int kSimplexCandidates = 16;   // vertices of the decision simplex
constexpr int kArmSlotCapacity = 16;
constexpr int kTeacherRequestSlices = 1;
constexpr int kTeacherResultSlices = 9;
constexpr uint32_t kTeacherWireVersion = 1;
constexpr uint32_t kWeightSnapshotMagic = 0x53574343u;   // "CCWS", little endian
constexpr uint64_t kCandidateSlotSentinel = ~0ull;

enum EventType : uint8_t {
  kWrite = 1, kQuery = 2, kReplayOutcome = 3, kArmJob = 4, kArmResult = 5,
  kTeacherRequest = 6, kTeacherResult = 7,
};
enum TeacherDtype : uint32_t { kNone = 0, kInt32 = 1, kFloat32 = 2, kFloat16 = 3, kBFloat16 = 4 };

#pragma pack(push, 1)
struct TensorSlice {                 // 40 B: where a tensor lives inside a payload region
  uint64_t offset_bytes, nbytes;
  uint32_t dtype, rank;
  uint32_t shape[4];
};

struct WriteEvent {                  // 568 B
  uint8_t event_type, source_rank, write_bucket, pad0[5];
  uint64_t candidate_id;             // (source_rank << 56) | per-rank sequence
  uint64_t gpu_step;
  uint64_t key_fp;                   // rolling fingerprint of the preceding tokens
  uint16_t key_rep[kKeyRepDim];      // fp16 bits
  uint16_t value_tok_ids[kSpanLength];
  uint32_t value_anchor_id;
  float pressure_at_write;
  float pre_write_ce;
  uint8_t pad1[4];
};

struct QueryEvent {                  // 736 B
  uint8_t event_type, source_rank, bucket, pad0[5];
  uint64_t query_id;
  uint64_t gpu_step;
  uint16_t query_rep[kKeyRepDim];
  float pressure;
  float pre_query_ce;
  uint64_t candidate_slot_ids[kSimplexCandidates];
  float candidate_cosines[kSimplexCandidates];
};

struct ReplayOutcome {               // 96 B
  uint8_t event_type, selected_rank, outcome_status, pad0[5];
  uint64_t replay_id, gpu_step, query_event_id, source_write_id;
  uint32_t slot_id, policy_version;
  uint64_t selection_step;
  float teacher_score, controller_logit, ce_before_replay, ce_after_replay, ce_delta_raw,
      bucket_baseline, reward_shaped, grad_cos_rare, grad_cos_total;
  uint16_t flags;
  uint8_t pad1[2];
};

struct ArmMaintenanceJob {           // 168 B
  uint8_t event_type, job_type, stream_id, flags;
  uint32_t slot_count;
  uint64_t job_id, frame_id, step, cache_read_cutoff;
  uint64_t slot_ids[kArmSlotCapacity];
};

struct ArmMaintenanceResult {        // 192 B
  uint8_t event_type, job_type, stream_id, status;
  uint32_t slot_count;
  uint64_t job_id, frame_id, step;
  uint32_t slots_scored, actions_confirmed, actions_rejected, pad0;
  float probe_seconds, oracle_seconds, cpu_seconds, frame_age_seconds;
  uint64_t slot_ids[kArmSlotCapacity];
};

struct TeacherRequest {              // 72 B
  uint8_t event_type, source_rank, status, flags;
  uint32_t slice_count;
  uint64_t request_id, step, weight_snapshot_version;
  TensorSlice full_ids;
};

struct TeacherResult {               // 456 B
  uint8_t event_type, source_rank, status, flags;
  uint32_t slice_count;
  uint64_t request_id, step, weight_snapshot_version, payload_version;
  float score_seconds, packet_seconds;
  uint32_t target_token_count, hidden_dim, plasticity_dim, fast_slow_mode, fast_slow_accepted;
  uint64_t fast_slow_step;
  float fast_slow_alpha, fast_slow_gate, fast_slow_effective_alpha;
  uint32_t fast_slow_reason, pad0;
  TensorSlice slices[kTeacherResultSlices];
};

struct WeightSnapshotHeader {        // 96 B
  uint32_t magic, wire_version, header_bytes, flags;
  uint64_t step, snapshot_version, total_bytes, checksum;
  uint32_t tensor_count, active_buffer, fast_slow_mode, fast_slow_accepted;
  uint64_t fast_slow_step;
  float fast_slow_alpha, fast_slow_gate, fast_slow_effective_alpha;
  uint32_t fast_slow_reason;
  uint64_t reserved0;
};
#pragma pack(pop)

static_assert(sizeof(TensorSlice) == 40, "wire: TensorSlice");
static_assert(sizeof(WriteEvent) == 568, "wire: WriteEvent");
static_assert(sizeof(QueryEvent) == 736, "wire: QueryEvent");
static_assert(sizeof(ReplayOutcome) == 96, "wire: ReplayOutcome");
static_assert(sizeof(ArmMaintenanceJob) == 168, "wire: ArmMaintenanceJob");
static_assert(sizeof(ArmMaintenanceResult) == 192, "wire: ArmMaintenanceResult");
static_assert(sizeof(TeacherRequest) == 72, "wire: TeacherRequest");
static_assert(sizeof(TeacherResult) == 456, "wire: TeacherResult");
static_assert(sizeof(WeightSnapshotHeader) == 96, "wire: WeightSnapshotHeader");
static_assert(offsetof(WriteEvent, key_rep) == 32 && offsetof(WriteEvent, value_tok_ids) == 544,
              "wire: WriteEvent field offsets");
static_assert(offsetof(QueryEvent, candidate_slot_ids) == 544, "wire: QueryEvent field offsets");

// Ring capacities used by the controller process.
constexpr std::size_t kWriteRingCapacity = 16384;
constexpr std::size_t kQueryRingCapacity = 16384;
constexpr std::size_t kReplayRingCapacity = 8192;

}  // namespace ccb::wire
