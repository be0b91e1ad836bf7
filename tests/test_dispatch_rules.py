"""The host-side rules that choose a kernel and its launch shape: pure functions of sizes, checked without a GPU."""
from flexengine_b200 import ops

SMS = 148                       # a B200's multiprocessors; on a device the functions ask the driver themselves
SLOTS = 6 * SMS                 # decode attention blocks resident at once


def test_decode_splits_stay_within_one_resident_round():
    for requests in (1, 2, 3, 5, 8, 13, 16, 31, 32, 64, 100, 256):
        for nkv in (1, 2, 4, 8):
            for ctx in (1, 31, 64, 500, 2048, 8192, 32768, 65536, 131072, 1 << 20):
                splits = ops.decode_splits(requests, nkv, ctx, SMS)
                tiles = -(-ctx // 32)
                assert 1 <= splits <= ops.DECODE_MAX_SPLITS, "the merge kernel's limit"
                assert splits == 1 or splits * 2 <= tiles, "a split walks at least two tiles"
                if requests * nkv <= SLOTS:
                    assert splits * requests * nkv <= SLOTS, (requests, nkv, ctx, splits)
    # the case that showed the fault: 28 splits of 32 pairs were 8 blocks more than fit
    assert ops.decode_splits(8, 4, 32768, SMS) == 27
    assert ops.decode_splits(8, 4, 2048, SMS) == 14 and ops.decode_splits(64, 4, 2048, SMS) == 3
    assert ops.decode_splits(1, 4, 2048, SMS) == 32
    # one request, one or two key/value heads, very long contexts: a round of the device would be more than the merge takes
    assert ops.decode_splits(1, 1, 32768, SMS) == ops.decode_splits(1, 2, 131072, SMS) == ops.DECODE_MAX_SPLITS
    with open(ops.__file__.replace("ops/__init__.py", "csrc/attention_mma.cu")) as f:
        assert f"MAX_SPLITS_SHARED = {ops.DECODE_MAX_SPLITS};" in f.read()


def test_cluster_splits_fit_one_round_of_the_device():
    # clusters resident at once by cluster size, as a B200 answered for the decode kernel at head size 128
    held = {2: 296, 3: 187, 4: 142, 5: 112, 6: 93, 7: 78, 8: 71, 9: 60, 10: 56, 11: 45, 12: 42, 13: 38, 14: 35, 15: 31, 16: 31}
    resident = held.__getitem__
    cluster = ops.decode_cluster_splits
    assert cluster(1, 2048, 32, resident) == 0                        # nothing to merge
    assert cluster(21, 4096, 32, resident) == 14                      # batch 8, four heads: 31 clusters of 16 fit, 32 are needed
    assert cluster(14, 2048, 32, resident) == 14
    assert cluster(13, 4096, 64, resident) == 8                       # batch 16: 60 clusters of 9 fit, 71 of 8
    assert cluster(64, 4096, 4, resident) == 16 and cluster(28, 4096, 16, resident) == 16      # few clusters: the largest
    assert cluster(6, 4096, 128, resident) == 6 and cluster(3, 4096, 256, resident) == 3       # many small ones: rounds anyway
    assert cluster(27, 8192, 32, resident) == 0 and cluster(111, 16384, 4, resident) == 0      # long contexts: two kernels
    assert cluster(12, 2048, 32, lambda s: 0) == 0                    # a device that places no such cluster
    assert cluster(21, 4096) == 16                                    # no word from the device: the kernel's limit
    for splits in range(1, 40):
        for clusters in (1, 4, 32, 64, 100, 256, 1000):
            got = cluster(splits, 2048, clusters, resident)
            assert 0 <= got <= min(splits, ops.DECODE_CLUSTER_MAX_SPLITS)


def test_prefill_splits_follow_the_work():
    def split(*a, **k):
        return ops.prefill_splits(*a, sms=SMS, **k)
    assert split([2048], [0], 28, 4) == 1                      # a whole prompt fills the device by itself
    assert split([64], [2048], 28, 4) == 8                     # 33 tiles: no split shorter than four
    assert split([64], [8192], 28, 4) == 18                    # eight blocks without splits; one round of the device
    assert split([2], [100000], 28, 4) == 32                   # never more than the merge takes
    assert split([64], [0], 28, 4) == 1 and split([40, 1, 1], [10, 20, 30], 4, 2) == 1
    assert split([16], [900], 28, 4) == 1 and split([16], [1010], 28, 4) == 4      # from sixteen tiles on
    assert split([64], [8192], 28, 4, window=256) == 1         # a window bounds what any row walks
    assert split([1] * 4 + [128], [500] * 4 + [4000], 28, 4) == 4      # decoded tokens beside a portion
    for lengths, starts in (([1], [0]), ([5, 700], [3, 9000]), ([128] * 4, [64000] * 4)):
        s = split(lengths, starts, 12, 2)
        assert 1 <= s <= ops.PREFILL_MAX_SPLITS


def test_attention_kernel_choice():
    def ok(*a):
        return ops.tcgen05_attention_ok(*a, sms=SMS)
    assert ok(300, 4, 2, 128) and ok(2, 4, 2, 64) and not ok(4096, 4, 2, 96) and not ok(4096, 4, 2, 256)
    # very many requests with a few tokens each at short contexts: the lighter blocks of the mma.sync kernel
    assert not ok(8, 28, 4, 128, [8] * 256, [0] * 256) and not ok(64, 28, 4, 128, [1] * 60 + [64], [200] * 60 + [0])
    assert ok(32, 28, 4, 128, [32] * 64, [0] * 64) and ok(500, 28, 4, 128, [1] * 30 + [500], [2000] * 30 + [0])


def test_upcoming_hint_only_for_small_steps():
    import torch
    assert ops._upcoming(torch.zeros(4, 4), 8) == (None, 0)            # not a CUDA tensor: nothing to ask for
    assert ops._upcoming(None, 8) == (None, 0)


def test_entry_points_take_the_types_their_c_declarations_name():
    """The loader reads every ``extern "C"`` declaration of the sources; each entry point the Python side calls is
    among them, with one ctypes type per parameter, pointers as pointers and 64-bit integers as such."""
    import ctypes
    import re
    from flexengine_b200.ops import library
    declared = {}
    for group in library.GROUPS:
        declared.update(library.prototypes(group))
    with open(ops.__file__) as f:
        called = set(re.findall(r"\bfe_\w+", f.read()))
    assert called and called <= set(declared), called - set(declared)
    restype, args = declared["fe_paged_prefill_tcgen05"]
    assert restype is ctypes.c_int and len(args) == 24
    assert args[0] is ctypes.c_void_p and args[1] is ctypes.c_longlong and args[17] is ctypes.c_float
    assert declared["fe_static_scratch_bytes"] == (ctypes.c_longlong, [])
    assert declared["fe_last_error"][0] is ctypes.c_char_p and declared["fe_set_pdl"] == (None, [ctypes.c_int])
