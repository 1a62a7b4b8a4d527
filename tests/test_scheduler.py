"""Host-side scheduler components (no GPU)."""
import pytest

from unillm_b200.scheduler import (AdaptivePolicyEngine, AdmissionController, AllocationEvent, CacheAwareAnalyzer,
                                   ChunkedPrefillConfig, ChunkedPrefillManager, ContinuousBatchingScheduler,
                                   GpuMemoryTracker, IntelligentScheduler, KvShape, PolicyAction, Request,
                                   RequestPriority, RequestState, ResourceLimits, SchedulerMetrics, SchedulingPolicy,
                                   StreamOverlapManager, StreamPriority, StreamType, create_compute_operation,
                                   create_h2d_operation)


def test_continuous_batching_budget_priority_and_no_drops():
    s = ContinuousBatchingScheduler(max_batch_size=3, max_sequence_length=100)
    ids = [s.add_request([1] * 20, 10), s.add_request([1] * 30, 10, RequestPriority.High),
           s.add_request([1] * 50, 10), s.add_request([1] * 5, 5), s.add_request([1] * 5, 5)]
    b = s.create_batch()
    assert [r.id for r in b.requests] == [ids[1], ids[0]]          # high priority first, then FIFO; 40+30 fits, +60 does not
    assert s.pending_count() == 3 and s.active_count() == 2         # every misfit went back to the queue
    assert b.total_tokens == 70 and b.is_prefill_batch
    s.update_request_state(ids[0], RequestState.Decoding)
    s.complete_request(ids[0]); s.fail_request(ids[1], "boom")
    assert s.get_stats().completed_requests == 1 and s.get_stats().failed_requests == 1
    with pytest.raises(Exception):
        s.complete_request(999)
    with pytest.raises(Exception):
        s.add_request([1] * 200, 10)
    b2 = s.create_batch()
    assert {r.id for r in b2.requests} == {ids[2], ids[3], ids[4]}


def test_chunked_prefill():
    m = ChunkedPrefillManager(ChunkedPrefillConfig(max_chunk_size=2048, chunking_threshold=4096))
    assert len(m.create_chunks(1, list(range(1000)))) == 1
    ids = m.create_chunks(2, list(range(5000)))
    assert len(ids) == 3
    spans = sorted((c.start_pos, c.end_pos) for c in m.get_active_chunks() if c.request_id == 2)
    assert spans == [(0, 2048), (2048, 4096), (4096, 5000)]          # contiguous, no recomputed overlap
    seen = []
    while True:
        nxt = m.get_next_chunk()
        if nxt is None:
            break
        seen.append((nxt[1].request_id, nxt[1].start_pos))
        m.complete_chunk(nxt[0])
    assert [p for r, p in seen if r == 2] == [0, 2048, 4096]
    assert m.is_request_complete(1) and m.is_request_complete(2) and m.get_stats().total_chunks_processed == 4
    m2 = ChunkedPrefillManager(ChunkedPrefillConfig(recompute_overlap=True))
    assert len(m2.create_chunks(1, list(range(5000)))) == 3


def test_stream_overlap_dependencies():
    m = StreamOverlapManager(streams_per_type=1)
    a = m.submit_operation(StreamType.H2D, StreamPriority.Normal, create_h2d_operation(1, 2, 4096), 0.001)
    b = m.submit_operation(StreamType.Compute, StreamPriority.High, create_compute_operation(7, (1, 1, 1), (128, 1, 1)), 0.002, [a])
    c = m.submit_operation(StreamType.H2D, StreamPriority.Low, create_h2d_operation(3, 4, 64), 0.001)
    started = m.schedule_operations()
    assert [op for op, _ in started] == [a]                        # b waits for a, c waits for the only H2D stream
    m.complete_operation(a)
    started = dict(m.schedule_operations())
    assert set(started) == {b, c} and m.active_count() == 2
    assert 0.0 < m.estimate_overlap_efficiency() < 1.0
    m.complete_operation(b); m.complete_operation(c)
    assert m.get_stats().completed_operations == 3 and m.pending_count() == 0


def test_intelligent_scheduler_policies_and_placement():
    cache = {tuple(range(64)): 64}
    lookup = lambda toks: 64 if tuple(toks[:64]) == tuple(range(64)) else 0
    kv = KvShape(num_layers=2, num_kv_heads=2, head_dim=16)
    s = IntelligentScheduler(max_batch_size=2, policy=SchedulingPolicy.LongestPrefixMatch, prefix_lookup=lookup, kv=kv, num_gpus=2)
    r1 = s.add_request(list(range(100, 200)), 10)
    r2 = s.add_request(list(range(64)) + [7] * 30, 10)
    r3 = s.add_request(list(range(300, 330)), 10)
    b = s.create_optimal_batch()
    assert b.requests[0].id in (r1, r2) and r2 in [r.id for r in b.requests] and s.pending_count() == 1
    s.optimizer.policy = SchedulingPolicy.GpuMemoryOptimized
    assert [r.id for r in s.create_optimal_batch().requests] == [r3]
    assert s.schedule_request(list(range(64)), 8).gpu_id == 0 and s.schedule_request([1, 2, 3], 8).gpu_id == 1
    s.complete_request(r2)
    assert s.get_comprehensive_stats().completed_requests == 1


def test_cache_analyzer_groups():
    a = CacheAwareAnalyzer(kv=KvShape(num_layers=1, num_kv_heads=1, head_dim=8))
    shared = list(range(40))
    reqs = [Request.new(1, shared + [1, 2], 4), Request.new(2, [9] * 50, 4), Request.new(3, shared + [5], 4),
            Request.new(4, shared[:10] + [3] * 40, 4)]
    ba = a.analyze_request_batch(reqs)
    assert len(ba.prefix_groups) == 1 and sorted(ba.prefix_groups[0].request_ids) == [1, 3]
    assert ba.prefix_groups[0].shared_prefix_length == 40 and ba.shared_memory_savings_bytes > 0
    res = a.optimize_batch_composition(reqs)
    ids = [r.id for r in reqs]
    assert abs(ids.index(1) - ids.index(3)) == 1 and res.groups == 1 and res.estimated_speedup > 1.0


def test_memory_tracker_and_admission():
    kv = KvShape(num_layers=1, num_kv_heads=1, head_dim=8, dtype_bytes=2)       # 32 B per token
    t = GpuMemoryTracker(total_memory=32 * 1000, kv=kv)
    reqs = [Request.new(i, [1] * 90, 10) for i in range(20)]
    f = t.can_accommodate_batch(reqs[:5])
    assert f.feasible and f.required == 5 * 100 * 32
    assert not t.can_accommodate_batch(reqs).feasible
    s = t.suggest_batch_size(reqs)
    assert 1 <= s.recommended <= s.max_feasible == 10 and s.memory_limited
    t.record_allocation(AllocationEvent(16000, 1)); t.record_allocation(AllocationEvent(12000, 2))
    st = t.get_memory_stats()
    assert st.used_memory == 28000 and st.watermark.value == "high" and st.memory_pressure > 0.5
    t.record_deallocation(16000, 1)
    assert t.get_memory_stats().available_memory == 20000
    ac = AdmissionController(ResourceLimits(max_concurrent_requests=2, max_total_tokens=300, max_memory_bytes=1 << 20), kv)
    assert ac.admit_request(1, 90, 10).admitted and ac.admit_request(2, 90, 10).admitted
    assert ac.admit_request(3, 90, 10, RequestPriority.Low).kind == "queued"
    assert ac.admit_request(4, 90, 10, RequestPriority.High).kind == "queued"
    assert ac.admit_request(5, 1000, 10).kind == "rejected"
    assert ac.complete_request(1) == [4]                             # the high-priority one leaves the queue first


def test_adaptive_policy_switches_on_cache_heavy_workload():
    e = AdaptivePolicyEngine(SchedulingPolicy.FCFS)
    d = None
    for _ in range(8):
        d = e.analyze_and_adapt(SchedulerMetrics(cache_hit_rate=0.9, memory_pressure=0.1, throughput_tokens_per_s=1000,
                                                 average_latency_ms=50, queue_length=4, policy=e.current))
    assert e.current == SchedulingPolicy.LongestPrefixMatch and d.workload.value == "cache_heavy"
    assert any(p.samples for p in e.get_policy_performance_summary())
