"""Variable-resolution video batching and the padded / grouped-length samplers."""
import random

from mindspeed_mm_b200.data.video_buckets import (GroupedLengthSampler, PaddedDistributedSampler, VariableVideoBatchSampler,
                                                   VideoBuckets, aspect_table, closest_aspect)


def test_aspect_table_and_bucket_choice():
    tab = aspect_table(854 * 480)
    assert all(h % 16 == 0 and w % 16 == 0 for h, w in tab.values())
    assert all(0.8 < h * w / (854 * 480) < 1.2 for h, w in tab.values())
    assert closest_aspect(480, 854, tab) == "0.56" and closest_aspect(854, 480, tab) == "1.78"
    b = VideoBuckets({"240p": {1: (1.0, 32), 17: (1.0, 8), 65: (1.0, 2)}, "480p": {1: (1.0, 16), 33: (1.0, 4)}})
    assert b.bucket_of(100, 480, 854)[:2] == ("480p", 33)
    assert b.bucket_of(20, 480, 854)[:2] == ("240p", 17)           # too short for 480p's only video bucket -> next resolution
    assert b.bucket_of(1, 480, 854)[:2] == ("480p", 1)
    assert b.bucket_of(80, 240, 426)[:2] == ("240p", 65)
    assert b.bucket_of(80, 100, 100) is None                        # smaller than every pixel budget
    assert b.bucket_of(10, 240, 426) is None                        # shorter than every frame count
    t, h, w = b.thw(("480p", 33, "0.56"))
    assert t == 33 and (h, w) == tab["0.56"] and b.batch_size(("480p", 33, "0.56")) == 4
    # keep probability thins a bucket: about half of the clips fall through to the next one
    thin = VideoBuckets({"240p": {17: (1.0, 8)}, "480p": {33: (0.5, 4)}})
    hits = [thin.bucket_of(100, 480, 854, seed=i * 7)[0] for i in range(400)]
    assert 120 < hits.count("480p") < 280 and hits.count("240p") == 400 - hits.count("480p")


def _meta(n, seed=0):
    rnd = random.Random(seed)
    shapes = [(100, 480, 854), (40, 480, 854), (1, 480, 854), (70, 240, 426), (20, 426, 240)]
    return [rnd.choice(shapes) for _ in range(n)]


def test_variable_video_sampler_batches_resume_and_rank_split():
    cfg = {"240p": {1: (1.0, 6), 17: (1.0, 4), 65: (1.0, 2)}, "480p": {1: (1.0, 3), 33: (1.0, 2)}}
    meta = _meta(97)
    world = 2
    per_rank = []
    for r in range(world):
        s = VariableVideoBatchSampler(meta, VideoBuckets(cfg), r, world, seed=3)
        per_rank.append(list(s))
        assert len(per_rank[-1]) == len(s)
    assert len(per_rank[0]) == len(per_rank[1]) > 5
    seen = set()
    for batches in per_rank:
        for mb in batches:
            assert len({(t, h, w) for _, t, h, w in mb}) == 1        # one shape per micro-batch
            _, t, h, w = mb[0]
            for i, *_ in mb:
                T, H, W = meta[i]
                assert T >= t and H * W >= 0.8 * h * w * 0.8         # target never exceeds what the clip offers
                seen.add(i)
    assert len(seen) == len(meta)                                    # nothing dropped (padding repeats, never removes)
    # resume after 3 steps gives the remaining stream
    s = VariableVideoBatchSampler(meta, VideoBuckets(cfg), 1, world, seed=3)
    it = iter(s)
    first = [next(it) for _ in range(3)]
    state = s.state_dict()
    assert state["consumed"] == 3 * world and first == per_rank[1][:3]
    s2 = VariableVideoBatchSampler(meta, VideoBuckets(cfg), 1, world, seed=3)
    s2.load_state_dict(state)
    assert list(s2) == per_rank[1][3:]
    # next epoch reshuffles
    assert list(s2) != per_rank[1] and s2.epoch == 2
    # drop_last never pads
    d = VariableVideoBatchSampler(meta, VideoBuckets(cfg), 0, 1, seed=3, drop_last=True)
    flat = [i for mb in d for i, *_ in mb]
    assert len(flat) == len(set(flat))


def test_padded_distributed_sampler_covers_everything_and_resumes():
    got = [list(PaddedDistributedSampler(10, r, 4, seed=1)) for r in range(4)]
    assert all(len(g) == 3 for g in got) and set(sum(got, [])) == set(range(10))
    s = PaddedDistributedSampler(10, 2, 4, seed=1)
    it = iter(s)
    a = next(it)
    st = s.state_dict()
    s2 = PaddedDistributedSampler(10, 2, 4, seed=1)
    s2.load_state_dict(st)
    assert [a] + list(s2) == got[2]
    tiny = [list(PaddedDistributedSampler(2, r, 4, shuffle=False)) for r in range(4)]
    assert sum(tiny, []) == [0, 1, 0, 1]
    assert len(list(PaddedDistributedSampler(10, 0, 4, drop_last=True))) == 2


def test_grouped_length_sampler_keeps_tasks_apart_and_lengths_close():
    rnd = random.Random(0)
    kinds = ["t2i"] * 70 + ["edit"] * 50
    lengths = [rnd.randint(10, 2000) for _ in kinds]
    bs, world, acc = 2, 2, 2
    own = [list(GroupedLengthSampler(kinds, lengths, bs, r, world, acc, seed=5, window=2)) for r in range(world)]
    unit = bs * world * acc
    assert len(own[0]) == len(own[1]) == (70 // unit * unit + 50 // unit * unit) // world
    assert not set(own[0]) & set(own[1])
    steps = len(own[0]) // bs
    spreads = []
    for s in range(0, steps, acc):                                   # one accumulation window = one task
        ids = [i for r in range(world) for i in own[r][s * bs:(s + acc) * bs]]
        assert len({kinds[i] for i in ids}) == 1
    for s in range(steps):
        ids = [i for r in range(world) for i in own[r][s * bs:(s + 1) * bs]]
        spreads.append(max(lengths[i] for i in ids) - min(lengths[i] for i in ids))
    assert sum(spreads) / len(spreads) < 500                         # random global batches would spread ~1200
    a = list(GroupedLengthSampler(kinds, lengths, bs, 0, world, acc, seed=5))
    b = list(GroupedLengthSampler(kinds, lengths, bs, 0, world, acc, seed=5))
    assert a == b
