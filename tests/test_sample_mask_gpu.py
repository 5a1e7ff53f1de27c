"""The mask sampler kernel: format (sorted, distinct, exact count), reproducibility, uniformity, and
bit-exact agreement with a numpy restatement of its algorithm (Philox-4x32-10 keys, keep the
`count` smallest, ties in channel order)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85


def philox_keys(lists, channels, seed):
    """keys[list, channel] as the kernel draws them: counter (channel // 4, list, 0, 0), key = seed."""
    q = np.arange((channels + 3) // 4, dtype=np.uint64)
    c = [np.broadcast_to(q, (lists, q.size)).copy(),
         np.broadcast_to(np.arange(lists, dtype=np.uint64)[:, None], (lists, q.size)).copy(),
         np.zeros((lists, q.size), np.uint64), np.zeros((lists, q.size), np.uint64)]
    k0, k1 = np.uint64(seed & 0xFFFFFFFF), np.uint64((seed >> 32) & 0xFFFFFFFF)
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(M0) * c[0]
        p1 = np.uint64(M1) * c[2]
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
        k0 = (k0 + np.uint64(W0)) & mask
        k1 = (k1 + np.uint64(W1)) & mask
    keys = np.stack(c, axis=-1).reshape(lists, -1)[:, :channels]
    return keys.astype(np.uint32)


def expected_lists(lists, channels, count, seed):
    keys = philox_keys(lists, channels, seed)
    order = np.argsort(keys, axis=1, kind="stable")        # ties: lower channel first
    return np.sort(order[:, :count], axis=1).astype(np.int32)


def draw(S, G, channels, count, seed):
    from sortnet_b200 import norm_dist_cuda as C
    out = torch.full((S, G, count), -1, dtype=torch.int32, device="cuda")
    C.sample_mask_into(out, channels, seed)
    return out.cpu().numpy()


@pytest.mark.parametrize("S,G,channels,count", [(16, 1, 5120, 4608), (3, 2, 50, 40), (4, 1, 12288, 11000),
                                                (2, 3, 37, 1), (5, 1, 1023, 1023), (1, 1, 7, 3)])
def test_matches_the_restated_algorithm(S, G, channels, count):
    seed = 0x1234567890ABCDEF + channels
    got = draw(S, G, channels, count, seed)
    assert np.array_equal(got.reshape(S * G, count), expected_lists(S * G, channels, count, seed))
    assert (np.diff(got, axis=-1) > 0).all() and got.min() >= 0 and got.max() < channels
    again = draw(S, G, channels, count, seed)
    assert np.array_equal(got, again)
    if count < channels:
        assert not np.array_equal(got, draw(S, G, channels, count, seed + 1))


def test_uniform_over_channels():
    lists, channels, count = 4096, 96, 24
    got = draw(lists, 1, channels, count, 99).reshape(lists, count)
    freq = np.bincount(got.ravel(), minlength=channels) / lists
    sigma = np.sqrt(0.25 * 0.75 / lists)
    assert np.abs(freq - 0.25).max() < 5 * sigma
    # channels 0 and 1 are kept together about count*(count-1)/(channels*(channels-1)) of the time
    both = (np.isin(0, got[:, :1]) if False else ((got == 0).any(1) & (got == 1).any(1))).mean()
    want = count * (count - 1) / (channels * (channels - 1))
    assert abs(both - want) < 5 * np.sqrt(want * (1 - want) / lists)


def test_layer_level_sampler_is_reproducible_and_sorted():
    from sortnet_b200.layers import sample_mask
    torch.manual_seed(5)
    a = sample_mask(4, 2, 300, 0.8, "cuda")
    torch.manual_seed(5)
    b = sample_mask(4, 2, 300, 0.8, "cuda")
    assert a.dtype == torch.int32 and a.dim() == 3 and a.shape[:2] == (4, 2)
    assert torch.equal(a, b)
    assert bool((a[..., 1:] > a[..., :-1]).all()) and int(a.min()) >= 0 and int(a.max()) < 300
    assert abs(a.size(-1) - 240) < 40
    c = sample_mask(4, 2, 300, 0.8, "cuda", count=17)
    assert c.shape == (4, 2, 17)


def test_batched_launch_writes_the_lists_of_the_separate_calls():
    """snb_sample_mask_batch: several (channels, count, seed) jobs in one launch, each bit-identical to
    its own snb_sample_mask call and to the restated algorithm."""
    from sortnet_b200 import norm_dist_cuda as C
    jobs = [(3072, 2750, 11), (5120, 4608, 12), (5120, 4590, 13), (40, 1, 14), (12288, 11000, 15)]
    S = 16
    outs = [torch.full((S, 1, count), -1, dtype=torch.int32, device="cuda") for _, count, _ in jobs]
    C.sample_masks_into(outs, [ch for ch, _, _ in jobs], [seed for _, _, seed in jobs])
    for out, (channels, count, seed) in zip(outs, jobs):
        assert np.array_equal(out.cpu().numpy(), draw(S, 1, channels, count, seed))
        assert np.array_equal(out.cpu().numpy().reshape(S, count), expected_lists(S, channels, count, seed))
    with pytest.raises(RuntimeError):
        C.sample_masks_into(outs[:2], [3072], [1, 2])
    with pytest.raises(RuntimeError):
        C.sample_masks_into([outs[0]] * 17, [3072] * 17, list(range(17)))    # more jobs than one launch takes


def test_model_masks_are_the_same_through_either_route():
    """SortMLPModel.draw_masks (one launch for all layers) against per-layer sample_mask calls with
    the same generator state."""
    from sortnet_b200 import layers
    model = layers.SortMLPModel(depth=4, width=256, input_dim=(1, 8, 8), num_classes=10, dropout=0.9).cuda()
    torch.manual_seed(21)
    batched = model.draw_masks(96, "cuda")
    torch.manual_seed(21)
    todo = [(k, l) for k, l in enumerate(model.fc_dist[1:]) if l.keep_rate != 1.0]
    counts = [int((torch.rand(l.in_features) < l.keep_rate).sum()) for _, l in todo]
    for (k, l), c in zip(todo, counts):
        single = layers.sample_mask(3, 1, l.in_features, l.keep_rate, "cuda", count=max(c, 1))
        assert torch.equal(batched[k], single)


def test_bad_arguments():
    from sortnet_b200 import norm_dist_cuda as C
    out = torch.empty(2, 1, 10, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError):
        C.sample_mask_into(out, 5, 1)              # more elements than channels
    with pytest.raises(RuntimeError):
        C.sample_mask_into(out.float(), 50, 1)     # wrong dtype


def test_check_index_lists_flags_bad_entries_and_order():
    """The debug validation of caller-made index lists (snb_check_index_lists)."""
    from sortnet_b200 import norm_dist_cuda as C
    good = torch.tensor([[[0, 3, 7, 9]], [[1, 2, 3, 4]]], dtype=torch.int32, device="cuda")
    assert C.check_index_lists(good, 10) is True
    unsorted = torch.tensor([[[0, 7, 3, 9]], [[1, 2, 3, 4]]], dtype=torch.int32, device="cuda")
    assert C.check_index_lists(unsorted, 10) is False
    repeated = torch.tensor([[[0, 3, 3, 9]]], dtype=torch.int32, device="cuda")
    assert C.check_index_lists(repeated, 10) is False
    for bad in ([[[0, 3, 7, 10]]], [[[-1, 3, 7, 9]]]):
        with pytest.raises(RuntimeError, match="outside"):
            C.check_index_lists(torch.tensor(bad, dtype=torch.int32, device="cuda"), 10)
    # the last entry of one list may exceed the first of the next
    two = torch.tensor([[[5, 9]], [[0, 1]]], dtype=torch.int32, device="cuda")
    assert C.check_index_lists(two, 10) is True


def test_debug_mode_validates_index_lists_before_the_kernels(monkeypatch):
    from sortnet_b200 import norm_dist_cuda as C
    monkeypatch.setattr(C, "DEBUG_INDEX_CHECKS", True)
    x = torch.rand(32, 3, 1, device="cuda")
    w = torch.randn(6, 5, device="cuda")
    y = torch.empty(32, 2, 1, device="cuda")
    pos = torch.empty(32, 2, 1, device="cuda", dtype=torch.int32)
    ci = torch.tensor([[[0, 2, 4]]], dtype=torch.int32, device="cuda")
    co = torch.tensor([[[1, 5]]], dtype=torch.int32, device="cuda")
    C.inf_dist_forward(x, w, y, pos, 1, ci, co)
    bad_ci = torch.tensor([[[0, 2, 5]]], dtype=torch.int32, device="cuda")      # w has 5 columns
    with pytest.raises(RuntimeError, match="w_index_ci"):
        C.inf_dist_forward(x, w, y, pos, 1, bad_ci, co)
    bad_co = torch.tensor([[[1, 6]]], dtype=torch.int32, device="cuda")         # w has 6 rows
    with pytest.raises(RuntimeError, match="w_index_co"):
        C.inf_dist_forward(x, w, y, pos, 1, ci, bad_co)
    # the ascending-list entry also checks its promise
    C.inf_dist_forward_sorted(x, w, y, pos, ci, co)
    unsorted = torch.tensor([[[2, 0, 4]]], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="ascending"):
        C.inf_dist_forward_sorted(x, w, y, pos, unsorted, co)
