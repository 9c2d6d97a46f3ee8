"""Host-side step metadata of the paged layout (gaac_b200/vllm/metadata.py, the entry construction of the reference's vLLM builder,
gaac/vllm/backend.py:205-254) on CPU: against a token-by-token restatement, and end to end through the oracle's paged store."""
import numpy as np
import torch
from oracle import gaac_oracle as O
from gaac_b200.vllm import metadata as M


def _entries_token_by_token(qsl, start):
    """One token at a time: consecutive tokens of a request that fall into the same block extend the current entry."""
    out = []
    for r in range(len(qsl) - 1):
        cur = None
        for i in range(qsl[r + 1] - qsl[r]):
            pos = start[r] + i
            if cur is not None and pos // 16 == cur[4]:
                cur[3] += 1
            else:
                cur = [qsl[r] + i, qsl[r] + i, pos % 16, 1, pos // 16]
                out.append(cur)
    return np.array([c[:4] for c in out], np.int32).reshape(-1, 4)


def test_entries_match_token_by_token_model():
    rng = np.random.default_rng(0)
    cases = [([0, 1, 2, 3], [15, 16, 31]), ([0, 37], [0]), ([0, 5, 5, 40], [11, 3, 16]), ([0], [])]
    for _ in range(30):
        R = int(rng.integers(1, 9))
        qlen = rng.integers(1, 70, R) * (rng.random(R) < 0.6) + 1 * (rng.random(R) >= 0) * 0
        qlen = np.where(qlen == 0, 1, qlen)
        cases.append((np.concatenate([[0], np.cumsum(qlen)]).tolist(), rng.integers(0, 200, R).tolist()))
    for qsl, start in cases:
        got = M.build_entries(qsl, start)
        want = _entries_token_by_token(qsl, start)
        assert got.dtype == np.int32 and np.array_equal(got, want), (qsl, start)
        assert int(got[:, 3].sum()) == qsl[-1]                                   # every query token is stored exactly once
        assert ((got[:, 2] + got[:, 3]) <= 16).all() and (got[:, 3] >= 1).all()


def test_context_pairs_cover_the_cached_tokens():
    ctx, new = [0, 37, 16, 100], [5, 3, 20, 1]
    d = M.build_context_pairs(ctx, new)
    assert d["cu_k"].tolist() == [0, 5, 45, 81, 182] and d["rows"] == 182 and d["max_k"] == 101
    # pairs of request 1: blocks 0, 1, 2 with 16, 16, 5 valid rows at scratch rows 5, 21, 37
    p1 = d["pairs"][d["owner"] == 1]
    assert p1.tolist() == [[0, 5, 16], [1, 21, 16], [2, 37, 5]]
    assert (d["owner"] == 0).sum() == 0 and d["pairs"][d["owner"] == 3][:, 2].sum() == 100
    # new tokens land right behind their request's context rows
    assert d["slots"].tolist()[:5] == [0, 1, 2, 3, 4] and d["slots"].tolist()[5:8] == [42, 43, 44] and d["slots"][-1] == 181


def test_entries_drive_the_paged_store_model_over_prefill_chunks_and_decode_steps():
    """Three requests: chunked prefill (two chunks), a whole-prompt prefill and decode steps, all through build_entries; what the
    oracle's store holds afterwards decodes to exactly the tokens that were written."""
    n_kv, num_blocks = 2, 64
    cal = {k: O.calibrate(O.synth_kv(k[0], n_kv, 512, 3), n_kv) for k in ("k", "v")}
    bases = {"k3": cal["k"][0], "k4": cal["k"][1], "v3": cal["v"][0], "v4": cal["v"][1]}
    st = O.PagedStoreModel(num_blocks, n_kv, raw_tiles=32, bases=bases, ovf_slot=128)
    rng = np.random.default_rng(1)
    blocks = rng.permutation(num_blocks)
    table = {0: blocks[0:8], 1: blocks[8:16], 2: blocks[16:24]}
    cached = {0: 0, 1: 0, 2: 0}
    hist = {r: (np.zeros((0, n_kv, 128), np.uint16), np.zeros((0, n_kv, 128), np.uint16)) for r in table}
    stream = {r: (O.synth_kv("k", n_kv, 512 + 120, 3)[:, 512:].transpose(1, 0, 2), O.synth_kv("v", n_kv, 512 + 120, 3)[:, 512:].transpose(1, 0, 2)) for r in table}
    schedule = [{0: 20, 1: 37}, {0: 13, 2: 16}] + [{0: 1, 1: 1, 2: 1}] * 30
    for step in schedule:
        reqs = sorted(step)
        qlen = [step[r] for r in reqs]
        qsl = np.concatenate([[0], np.cumsum(qlen)])
        start = [cached[r] for r in reqs]
        key = np.concatenate([np.roll(stream[r][0], r, axis=0)[cached[r]:cached[r] + step[r]] for r in reqs])
        val = np.concatenate([np.roll(stream[r][1], r, axis=0)[cached[r]:cached[r] + step[r]] for r in reqs])
        slot_mapping = np.concatenate([table[r][(cached[r] + np.arange(step[r])) // 16] * 16 + (cached[r] + np.arange(step[r])) % 16 for r in reqs])
        ent = M.build_entries(qsl, start)
        ent = M.resolve_blocks(torch.from_numpy(ent), torch.from_numpy(slot_mapping)).numpy()
        st.store(key, val, ent)
        for i, r in enumerate(reqs):
            hist[r] = (np.concatenate([hist[r][0], key[qsl[i]:qsl[i + 1]]]), np.concatenate([hist[r][1], val[qsl[i]:qsl[i + 1]]]))
            cached[r] += step[r]
    assert st.err == 0
    for r in table:
        L = cached[r]
        for kind, want in (("k", hist[r][0]), ("v", hist[r][1])):
            for kvh in range(n_kv):
                got = np.concatenate([st.decode_tile(int(table[r][b]), kvh, kind) for b in range((L + 15) // 16)])[:L]
                assert np.array_equal(got, want[:, kvh]), (r, kind, kvh)


def test_entry_uploader_keeps_inactive_rows_inactive():
    up = M.EntryUploader(max_entries=8, n_kv=2, device="cpu")
    ent, freeq = up.upload(M.build_entries([0, 1, 2, 3], [5, 15, 16]), torch.arange(3) * 16 + torch.tensor([5, 15, 0]))
    assert ent.shape == (3, 4) and freeq.numel() == 3 * 4 and ent[:, 0].tolist() == [0, 1, 2]
    assert up.ent[3:, 0].tolist() == [-1] * 5 and ent.data_ptr() == up.ent.data_ptr()
    big, fq = up.upload(np.zeros((9, 4), np.int32))
    assert big.shape == (9, 4) and big.data_ptr() != up.ent.data_ptr() and fq.numel() == 9 * 4
