"""The prover's random stream expanded on the device == the CPU generator (oracle restatement of zkp-core/src/rng.rs:279-417,
itself pinned by the three whole openings of the L5 corpus, whose pads and salts it draws): words and field elements from
any stream position, across 64-byte pieces and 8 KiB blocks; then a hiding commitment whose pads and salts never exist on
the host, equal to the CPU commitment drawn from the same generator in the reference's order (pcs.rs:733-745, 788-792).
Byte work: bit-exact."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from intelligenceregulation_b200 import backend

    d = backend.B200Backend(device=0)
    yield d
    d.ctx.close()


@pytest.mark.parametrize("skip_words,count", [(0, 1), (0, 4096), (3, 1000), (1019, 40), (7, 9), (1024 * 5 + 1, 3000), (0, 2504 * 280)])
def test_field_draws_from_any_position(dev, oracle, skip_words, count):
    r = oracle.ZkRng(1234 + skip_words, b"b200-rng")
    for _ in range(skip_words):
        r.next_u64()
    assert r.words_consumed == skip_words
    key = r.key
    want = r.fp_vec(count)
    assert (dev.ctx.rng_fill(key, skip_words, count, True) == want).all()
    assert r.words_consumed == skip_words + 2 * count


def test_word_draws_and_salts(dev, oracle):
    r = oracle.ZkRng(99, b"b200-rng-words")
    key = r.key
    r.fp()  # two words gone
    salts = r.salts(777)  # 4 words each
    got = dev.ctx.rng_fill(key, 2, 4 * 777, False)
    assert got.view(np.uint8).reshape(777, 32).tobytes() == salts.tobytes()
    nxt = dev.ctx.rng_fill(key, r.words_consumed, 5, False)
    assert [int(x) for x in nxt] == [r.next_u64() for _ in range(5)]


def test_commitment_with_pads_and_salts_drawn_on_the_device(dev, oracle):
    import torch

    o = oracle
    torch.cuda.set_device(0)
    log_cols, ir, rows, q = 10, 4, 200, 64
    n, nn = 1 << log_cols, (1 << log_cols) * ir
    tag = o.HashTag.for_profile("hashline-zk-mr1/b200-rng/1")
    data = o.ZkRng(5, b"data").fp_vec(rows * n)
    cpu = o.commit_zk(o.PcsParams(log_cols, ir, 8), data, 12, q, o.ZkRng(6, b"commit"), tag)
    # the same generator, expanded on the device: pads = fp_vec(rows * q), then nn salts (pcs.rs:788-792)
    g = o.ZkRng(6, b"commit")
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    dev.ctx.set_stream(stream.cuda_stream)
    d_data = torch.from_numpy(data.view(np.int64)).cuda()
    d_pows = torch.from_numpy(o.coset_powers(7, nn).view(np.int64)).cuda()
    d_pads = torch.empty(rows * q, dtype=torch.int64, device="cuda")
    d_salts = torch.empty(nn * 32, dtype=torch.uint8, device="cuda")
    d_levels = torch.empty((2 * nn - 1) * 32, dtype=torch.uint8, device="cuda")
    dev.ctx.rng_fill_dev(g.key, 0, rows * q, True, d_pads.data_ptr())
    dev.ctx.rng_fill_dev(g.key, 2 * rows * q, 4 * nn, False, d_salts.data_ptr())
    st = dev.commit_zk_dev(log_cols, ir, d_data.data_ptr(), rows, d_pads.data_ptr(), q, d_pows.data_ptr(), tag.column)
    st.merkle_dev(d_salts.data_ptr(), tag.leaf, tag.node, d_levels.data_ptr())
    torch.cuda.synchronize()
    assert bytes(d_levels[-32:].cpu().numpy()) == cpu.root
    assert (d_pads.cpu().numpy().view(np.uint64) == cpu.pads).all()
    st.free()
    dev.ctx.set_stream(0)
