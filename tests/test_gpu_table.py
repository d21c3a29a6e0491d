"""Expert table: device generator == host generator, repack round trip, bit-exact dequant
(reference src/quant.c:82-105, 147-175, 216-247), tensor-parallel shard geometry."""
import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small(fb):
    d = fb.MoeDecoder(3, 512, 512, 8, 2, True, [H.Q6, H.Q4, H.Q5])
    d.generate(11)
    yield d
    d.close()


@pytest.mark.parametrize("layer", [0, 1, 2])
@pytest.mark.parametrize("expert", [0, 5, 8])
def test_generated_bytes_match_host_generator(fb, small, layer, expert):
    dt = small.down_types[layer]
    for m, (t, rows, cols) in ((fb.M_GATE, (H.Q4, 512, 512)), (fb.M_UP, (H.Q4, 512, 512)), (fb.M_DOWN, (dt, 512, 512))):
        dev = small.export_shard(layer, expert, m)
        host = fb.synth_matrix(11, layer, expert, m, t, rows, cols)
        assert dev.size == host.size
        assert (dev == host).all()


@pytest.mark.parametrize("layer", [0, 1, 2])
def test_dequant_bit_exact(fb, small, oracle, layer):
    dt = small.down_types[layer]
    for m, t in ((fb.M_GATE, H.Q4), (fb.M_DOWN, dt)):
        got = small.dequant_shard(layer, 3, m)
        raw = fb.synth_matrix(11, layer, 3, m, t, 512, 512)
        rb = fb.matrix_bytes(t, 1, 512)
        for r in range(0, 512, 37):
            want = oracle.dequantize(raw[r * rb:(r + 1) * rb], t, 512)
            assert (H.bits(got[r]) == H.bits(want)).all(), (layer, m, r)


def test_upload_repack_round_trip(fb, small):
    rng = np.random.default_rng(5)
    for layer in (0, 1, 2):
        rec = rng.integers(0, 256, small.record_bytes(layer), dtype=np.uint8)
        small.upload_expert(layer, 2, rec)
        gb = fb.matrix_bytes(H.Q4, 512, 512)
        assert (small.export_shard(layer, 2, fb.M_GATE) == rec[:gb]).all()
        assert (small.export_shard(layer, 2, fb.M_UP) == rec[gb:2 * gb]).all()
        assert (small.export_shard(layer, 2, fb.M_DOWN) == rec[2 * gb:]).all()
    small.generate(11)


@pytest.mark.parametrize("tp", [2])
def test_tp_shards_are_slices(fb, tp):
    n_embd, inter = 512, 1024
    for rank in range(tp):
        d = fb.MoeDecoder(1, n_embd, inter, 4, 2, True, [H.Q6], tp_rank=rank, tp_size=tp)
        d.generate(3)
        il = inter // tp
        full_g = fb.synth_matrix(3, 0, 1, fb.M_GATE, H.Q4, inter, n_embd).reshape(inter, -1)
        assert (d.export_shard(0, 1, fb.M_GATE).reshape(il, -1) == full_g[rank * il:(rank + 1) * il]).all()
        full_d = fb.synth_matrix(3, 0, 1, fb.M_DOWN, H.Q6, n_embd, inter).reshape(n_embd, inter // 256, 210)
        bl = il // 256
        assert (d.export_shard(0, 1, fb.M_DOWN).reshape(n_embd, bl, 210) == full_d[:, rank * bl:(rank + 1) * bl]).all()
        d.close()


def test_full_shape_table_sample(fb, oracle):
    """397B shape, one layer of 16 experts: bytes and dequant of sampled rows."""
    d = fb.MoeDecoder(1, 4096, 1024, 16, 10, True, [H.Q6])
    d.generate(21)
    assert d.record_bytes(0) == 8159232
    for e in (0, 9, 16):
        for m, (t, rows, cols) in ((fb.M_UP, (H.Q4, 1024, 4096)), (fb.M_DOWN, (H.Q6, 4096, 1024))):
            host = fb.synth_matrix(21, 0, e, m, t, rows, cols)
            assert (d.export_shard(0, e, m) == host).all()
            got = d.dequant_shard(0, e, m)
            rb = fb.matrix_bytes(t, 1, cols)
            for r in (0, 1, rows // 2 + 3, rows - 1):
                want = oracle.dequantize(host[r * rb:(r + 1) * rb], t, cols)
                assert (H.bits(got[r]) == H.bits(want)).all()
    d.close()


def test_load_expert_store_written_by_the_reference(fb, ref, tmp_path):
    """A .qmoe file written by the reference's own writer (src/expert_store.c:128-172, the layout of
    tools/prepare_experts.c:262-291) is read into the table: bytes of every routed expert match, the shared expert
    (not part of such files) is untouched, mismatching files are refused."""
    n_embd, inter, n_experts = 512, 256, 8
    dts = [H.Q6, H.Q5, H.Q4]
    recs = [(dt, [H.expert_record(fb, 900, l, e, dt, n_embd, inter) for e in range(n_experts)])
            for l, dt in enumerate(dts)]
    path = str(tmp_path / "experts.qmoe")
    ref.write_store(path, recs)
    d = fb.MoeDecoder(2, n_embd, inter, n_experts, 2, True, dts[1:])       # store layers 1 and 2
    d.generate(11)
    assert d.load_qmoe(path, first_store_layer=1) == 2 * n_experts
    gb = fb.matrix_bytes(H.Q4, inter, n_embd)
    for l in range(2):
        for e in (0, 3, n_experts - 1):
            rec = recs[1 + l][1][e]
            assert (d.export_shard(l, e, fb.M_GATE) == rec[:gb]).all()
            assert (d.export_shard(l, e, fb.M_UP) == rec[gb:2 * gb]).all()
            assert (d.export_shard(l, e, fb.M_DOWN) == rec[2 * gb:]).all()
        shared = fb.synth_matrix(11, l, n_experts, fb.M_DOWN, dts[1 + l], n_embd, inter)
        assert (d.export_shard(l, n_experts, fb.M_DOWN) == shared).all()
    with pytest.raises(RuntimeError):
        d.load_qmoe(path, first_store_layer=0)      # store layer 0 is Q6_K, the table's layer 0 is Q5_K
    with pytest.raises(RuntimeError):
        d.load_qmoe(path, first_store_layer=2)      # runs past the end of the file's layers
    with pytest.raises(RuntimeError):
        d.load_qmoe(str(tmp_path / "missing.qmoe"))
    d.close()
