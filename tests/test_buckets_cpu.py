from noeira_b200 import nn
from noeira_b200.parallel.buckets import BucketedReducer, GradMarks, plan_buckets


def test_marks_from_arena_and_bucket_plan():
    nn.manual_seed(0)
    blocks = [nn.Sequential(nn.Linear(16, 32), nn.Linear(32, 16)) for _ in range(4)]
    model = nn.Sequential(*blocks, nn.Linear(16, 4))
    opt = nn.Adam(model.named_params(), lr=1e-3)
    arena = opt.arenas[0] if hasattr(opt, "arenas") else opt.arena
    marks = GradMarks.from_arena(arena, lambda name: name.split(".")[0])
    assert [m.name for m in marks.marks] == ["0", "1", "2", "3", "4"]
    assert all(a.end <= b.begin for a, b in zip(marks.marks, marks.marks[1:]))
    per_block = marks.marks[0].end - marks.marks[0].begin
    buckets = plan_buckets(marks.marks, bucket_elems=2 * per_block - 8)
    # ready order: the small head ("4") + blocks 3 and 2 first, then blocks 1 + 0
    assert [b.units for b in buckets] == [("2", "3", "4"), ("0", "1")]
    assert buckets[0].ready_after == "2" and buckets[0].end == marks.marks[-1].end
    assert buckets[-1].begin == 0 and buckets[-1].ready_after == "0"
    calls = []
    red = BucketedReducer(buckets, lambda b, e: calls.append((b, e)))
    for unit in ("4", "3"):
        red.on_unit_done(unit)
    assert calls == []
    red.on_unit_done("2")
    assert calls == [(buckets[0].begin, buckets[0].end)]
    red.on_unit_done("1")
    assert len(calls) == 1
    red.finish()                                   # whatever backward did not announce is reduced at the end
    assert len(calls) == 2 and calls[-1][0] == 0
    covered = sorted(calls)
    assert covered[0][0] == 0 and covered[-1][1] == marks.marks[-1].end and covered[0][1] <= covered[1][0]   # alignment padding between units is not reduced
    one = plan_buckets(marks.marks, bucket_elems=1)
    assert [b.units for b in one] == [("4",), ("3",), ("2",), ("1",), ("0",)]


def test_bucket_waits_for_all_of_its_units_in_any_order():
    """Units of one bucket may finish in any order (token table before position table); the bucket leaves only after the
    last of them, and buckets leave in the planned order."""
    from noeira_b200.parallel.buckets import BucketedReducer, GradMarks, plan_buckets
    gm = GradMarks()
    for i in range(5):
        gm.add(f"u{i}", i * 100, (i + 1) * 100)
    buckets = plan_buckets(gm.marks, 200)            # {u3,u4}, {u1,u2}, {u0}
    assert [b.units for b in buckets] == [("u3", "u4"), ("u1", "u2"), ("u0",)]
    sent = []
    red = BucketedReducer(buckets, lambda b, e: sent.append((b, e)))
    red.on_unit_done("u4")
    assert sent == []
    red.on_unit_done("u1")                            # out of order: bucket 1 is not complete, bucket 0 neither
    assert sent == []
    red.on_unit_done("u3")
    assert sent == [(300, 500)]
    red.on_unit_done("u0")                            # complete, but bucket 1 has to go first
    assert sent == [(300, 500)]
    red.on_unit_done("u2")
    assert sent == [(300, 500), (100, 300), (0, 100)]
    red.finish()
    assert len(sent) == 3
    red.on_unit_done("u3")                            # next step starts clean
    assert len(sent) == 3
