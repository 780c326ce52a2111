"""Slot table: ids, dense storage, lifecycle, visibility, persistence -- one property per test (CPU)."""
import pytest
import torch

from chaoscontrol_b200.slot_table import (SLOT_ACTIVE, SLOT_QUARANTINED, SLOT_RETIRED, SLOT_WARMING, SlotRecord,
                                          SlotTable)


def _table(n=4, dim=3):
    t = SlotTable()
    ids = [t.append(torch.full((1, dim), float(i)), bucket_id=i % 2, event_id=10 + i, step=i) for i in range(n)]
    return t, ids


def test_ids_are_monotonic_and_never_reused():
    t, ids = _table(3)
    assert ids == [0, 1, 2]
    t.retire(1)
    assert t.append(torch.zeros(1, 3)) == 3 and 1 not in t.active_slot_ids()


def test_append_records_metadata():
    t, ids = _table(2)
    r = t.record(ids[1])
    assert isinstance(r, SlotRecord) and r.state == SLOT_WARMING and r.created_step == 1 and r.bucket_id == 1
    assert r.event_id == 11 and r.write_generation == 0 and len(t) == t.n_active == 2


def test_append_with_id_keeps_foreign_identity_and_advances_the_allocator():
    t = SlotTable()
    assert t.append_with_id(40, torch.ones(1, 2), generation=7, event_id=5) == 40
    assert t.record(40).write_generation == 7 and t.append(torch.zeros(1, 2)) == 41
    with pytest.raises(ValueError, match="already exists"):
        t.append_with_id(40, torch.ones(1, 2))


def test_append_rows_matches_repeated_append():
    rows = torch.arange(12.0).view(4, 3)
    a, b = SlotTable(), SlotTable()
    ids = a.append_rows(rows, [0, 1, 0, 1], [5, 6, 7, 8], step=3, survival=0.5)
    for i in range(4):
        b.append(rows[i], bucket_id=i % 2, event_id=5 + i, step=3, survival=0.5)
    assert ids == b.active_slot_ids() and torch.equal(a.slot_matrix(), b.slot_matrix())
    assert a.state_dict()["survival"] == b.state_dict()["survival"] and a.append_rows(rows[:0], [], []) == []


def test_storage_grows_past_the_first_reservation():
    t = SlotTable()
    for i in range(200):
        t.append(torch.full((1, 2), float(i)))
    m = t.slot_matrix()
    assert m.shape == (200, 2) and float(m[199, 0]) == 199.0 and float(m[0, 0]) == 0.0


def test_retire_single_compacts_rows_and_reindexes():
    t, ids = _table(4)
    assert t.retire(ids[1]) is True
    assert t.n_active == 3 and t.slot_matrix()[:, 0].tolist() == [0.0, 2.0, 3.0]
    assert [t.slot_id_to_physical(i) for i in (ids[0], ids[2], ids[3])] == [0, 1, 2]
    assert t.physical_to_slot_id(1) == ids[2] and t.slot_id_to_physical(ids[1]) is None and t.physical_to_slot_id(3) is None


def test_retire_many_ignores_unknown_and_duplicate_ids():
    t, ids = _table(4)
    assert t.retire_many([ids[3], 99, ids[0], ids[3]]) == [ids[3], ids[0]]
    assert t.slot_matrix()[:, 0].tolist() == [1.0, 2.0] and t.retire_many([99]) == [] and t.retire(99) is False


def test_retired_record_is_kept_until_purged():
    t, ids = _table(2)
    t.retire(ids[0], reason="distilled")
    r = t.record(ids[0])
    assert r.state == SLOT_RETIRED and r.retire_reason == "distilled" and r.write_generation == 1
    assert t.get_tensor(ids[0]) is None and ids[0] not in [x.slot_id for x in t.active_records()]
    assert t.purge_retired() == 1 and t.record(ids[0]) is None and t.purge_retired() == 0


def test_retire_everything_leaves_a_usable_table():
    t, ids = _table(3)
    t.retire_many(ids)
    assert t.n_active == 0 and t.slot_matrix().numel() == 0 and t.visible_indices() == []
    assert t.append(torch.ones(1, 3)) == 3 and t.slot_matrix().shape == (1, 3)


def test_quarantine_zeroes_priority_but_keeps_the_row_visible():
    t, ids = _table(3)
    assert t.priority_vector().tolist() == [1.0, 1.0, 1.0]
    assert t.quarantine(ids[1]) is True
    assert t.priority_vector().tolist() == [1.0, 0.0, 1.0] and t.visible_indices() == [0, 1, 2]
    r = t.record(ids[1])
    assert r.state == SLOT_QUARANTINED and r.quarantine_count == 1 and t.quarantine(99) is False


def test_release_restores_priority_and_state():
    t, ids = _table(2)
    t.quarantine(ids[0])
    assert t.release(ids[0]) is True and t.priority_vector().tolist() == [1.0, 1.0]
    assert t.record(ids[0]).state == SLOT_ACTIVE and t.release(99) is False


def test_priority_follows_rows_through_compaction():
    t, ids = _table(3)
    t.quarantine(ids[2])
    t.retire(ids[0])
    assert t.priority_vector().tolist() == [1.0, 0.0] and t.priority_vector([1]).tolist() == [0.0]
    assert t.priority_vector([]).numel() == 0


def test_every_lifecycle_mutation_bumps_the_generation():
    t, ids = _table(1)
    sid, gens = ids[0], []
    for op in (lambda: t.replace_tensor(sid, torch.ones(1, 3)), lambda: t.scale_survival(sid, 0.5),
               lambda: t.quarantine(sid), lambda: t.release(sid), lambda: t.retire(sid)):
        op()
        gens.append(t.record(sid).write_generation)
    assert gens == [1, 2, 3, 4, 5]


def test_replace_tensor_writes_in_place_and_probe_swaps_can_skip_the_bump():
    t, ids = _table(2)
    view = t.slot_matrix()
    assert t.replace_tensor(ids[1], torch.tensor([[7.0, 8.0, 9.0]])) is True
    assert view[1].tolist() == [7.0, 8.0, 9.0] and t.record(ids[1]).write_generation == 1
    t.replace_tensor(ids[1], torch.zeros(3), bump_generation=False)
    assert t.record(ids[1]).write_generation == 1 and float(t.get_tensor(ids[1]).abs().sum()) == 0.0
    assert t.replace_tensor(99, torch.zeros(3)) is False


def test_scale_survival_multiplies():
    t = SlotTable()
    sid = t.append(torch.zeros(1, 2), survival=2.0)
    t.scale_survival(sid, 0.9)
    t.scale_survival(sid, 0.5)
    assert t.state_dict()["survival"] == pytest.approx([0.9]) and t.scale_survival(99, 0.1) is False


def test_get_tensor_is_a_row_view():
    t, ids = _table(2)
    v = t.get_tensor(ids[0])
    assert v.shape == (1, 3)
    v.fill_(5.0)
    assert t.slot_matrix()[0].tolist() == [5.0, 5.0, 5.0]


def test_visibility_by_cutoff_and_bucket():
    t, ids = _table(4)                                              # event ids 10..13, buckets 0 1 0 1
    assert t.visible_indices(read_cutoff=11) == [0, 1] and t.visible_indices(read_cutoff=9) == []
    assert t.visible_indices(bucket_id=1) == [1, 3] and t.visible_indices(read_cutoff=12, bucket_id=0) == [0, 2]
    assert t.visible_indices(read_cutoff=None) == [0, 1, 2, 3]


def test_slot_matrix_subsets():
    t, ids = _table(5)
    full = t.slot_matrix()
    assert t.slot_matrix([1, 2, 3]).data_ptr() == full[1:4].data_ptr()          # a contiguous run stays a view
    gathered = t.slot_matrix([4, 0])
    assert gathered[:, 0].tolist() == [4.0, 0.0] and t.slot_matrix([]).numel() == 0
    assert t.slot_matrix(list(range(5))).data_ptr() == full.data_ptr()


def test_list_view_of_the_store():
    t, ids = _table(3)
    rows = t._slots
    assert len(rows) == 3 and rows[1].shape == (1, 3) and [r[0, 0].item() for r in rows] == [0.0, 1.0, 2.0]
    assert [r[0, 0].item() for r in rows[1:]] == [1.0, 2.0] and bool(rows)
    rows[2] = torch.full((1, 3), 9.0)
    assert t.slot_matrix()[2].tolist() == [9.0, 9.0, 9.0]
    t._slots = [torch.ones(1, 3), torch.zeros(1, 3)]
    assert t.n_active == 2 and not bool(SlotTable()._slots)


def test_state_round_trip_preserves_everything_live():
    t, ids = _table(4)
    t.quarantine(ids[1])
    t.scale_survival(ids[2], 0.5)
    t.retire(ids[0])
    u = SlotTable()
    u.load_state_dict(t.state_dict())
    assert torch.equal(u.slot_matrix(), t.slot_matrix()) and u.active_slot_ids() == t.active_slot_ids()
    assert u.priority_vector().tolist() == t.priority_vector().tolist()
    assert u.record(ids[1]).state == SLOT_QUARANTINED and u.record(ids[1]).write_generation == t.record(ids[1]).write_generation
    assert u.visible_indices(read_cutoff=12) == t.visible_indices(read_cutoff=12)
    assert u.append(torch.zeros(1, 3)) == 4                                       # the allocator resumes, no reuse


def test_state_dict_leaves_retired_records_out():
    t, ids = _table(2)
    t.retire(ids[0])
    assert set(t.state_dict()["records"]) == {ids[1]} and len(t.state_dict()["slots"]) == 1


def test_state_dict_without_priority_defaults_to_one():
    t, _ = _table(2)
    d = t.state_dict()
    del d["priority"]
    u = SlotTable()
    u.load_state_dict(d)
    assert u.priority_vector().tolist() == [1.0, 1.0]
