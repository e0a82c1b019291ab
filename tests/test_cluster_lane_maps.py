"""Lane arithmetic of the per-sample cluster kernel with eight outputs per thread
(csrc/persample_cluster8.cu), replayed with numpy on the CPU: the window / half assignment covers the
24x24 conv outputs exactly once, the 6x8 patches stay inside the image, the reduce-scatter of the
subsample-filter gradient lands every filter element on the lane that stores it, and the lanes that
send FC partial sums cover all ten outputs for all six CTAs."""
import numpy as np

LANES = np.arange(32)
COMPUTE_WARPS = 3
WINDOWS_PER_WARP = 12


def lane_geometry(warp, lane):
    slot, half = lane >> 1, lane & 1
    live = slot < WINDOWS_PER_WARP
    win = WINDOWS_PER_WARP * warp + slot if live else 35
    p, q = divmod(win, 6)
    return live, win, half, 4 * p + 2 * half, 4 * q


def test_outputs_are_covered_once_and_patches_fit():
    cover = np.zeros((24, 24), dtype=int)
    for warp in range(COMPUTE_WARPS):
        for lane in range(32):
            live, _, _, y0, x0 = lane_geometry(warp, lane)
            assert y0 + 5 <= 27 and x0 + 7 <= 27          # 6 rows x 8 columns of the 28x28 image
            assert (y0 * 28 + x0) % 4 == 0                # 128-bit shared-memory loads
            if live:
                cover[y0:y0 + 2, x0:x0 + 4] += 1
    assert (cover == 1).all()


def test_subsample_gradient_reduce_scatter_lands_on_the_storing_lane():
    rng = np.random.default_rng(0)
    half = LANES & 1
    live = (LANES >> 1) < WINDOWS_PER_WARP
    gs = rng.standard_normal((8, 32))
    gs[:, ~live] = 0.0
    terms = gs.copy()
    for keep_n in (4, 2, 1):
        mask = keep_n << 2
        upper = (LANES & mask) != 0
        nxt = gs.copy()
        for i in range(keep_n):
            send = np.where(upper, gs[i], gs[i + keep_n])
            keep = np.where(upper, gs[i + keep_n], gs[i])
            nxt[i] = keep + send[LANES ^ mask]
        gs = nxt
    total = gs[0] + gs[0][LANES ^ 2]
    stored = np.full(16, np.nan)
    for lane in range(32):
        if lane & 2:
            continue
        idx = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1)
        elem = (2 * (lane & 1) + (idx >> 2)) * 4 + (idx & 3)
        assert np.isnan(stored[elem])
        stored[elem] = total[lane]
    want = np.array([terms[(elem // 4 % 2) * 4 + elem % 4][half == elem // 8].sum() for elem in range(16)])
    assert np.allclose(stored, want)


def test_fc_partial_sums_reach_every_cta():
    """A window's two lanes split the ten outputs (lane half h takes k = 5h .. 5h+4); after the
    butterfly over the warp's windows lane 2c + h holds those five sums and stores them into CTA c's
    buffer row of 16 floats at [8h .. 8h+4] (one 16-byte and one 4-byte one-way store); the receiver's
    lane k < 10 reads slot k (k < 5) or k + 3."""
    rng = np.random.default_rng(1)
    half = LANES & 1
    live = (LANES >> 1) < WINDOWS_PER_WARP
    pk = rng.standard_normal((5, 32))
    pk[:, ~live] = 0.0
    terms = pk.copy()
    for m in (2, 4, 8, 16):
        pk = pk + pk[:, LANES ^ m]
    want = np.array([terms[k % 5][half == k // 5].sum() for k in range(10)])
    row = np.full((6, 16), np.nan)
    stores = 0
    for lane in range(12):
        c, h = lane >> 1, lane & 1
        assert (8 * h * 4) % 16 == 0                      # the 16-byte store is aligned
        row[c][8 * h:8 * h + 4] = pk[0:4, lane]
        row[c][8 * h + 4] = pk[4][lane]
        stores += 2
    got = np.array([[row[c][k if k < 5 else k + 3] for k in range(10)] for c in range(6)])
    assert np.allclose(got, want[None, :])
    assert stores == 24                                   # per warp; 60 with one store per float
    # bytes counted on a receiver's mbarrier per sample: 6 CTAs x 3 warps x 10 floats
    assert 6 * COMPUTE_WARPS * 10 * 4 == 720
