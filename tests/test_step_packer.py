"""Host-only checks of the step packer: layout of the packed int32 metadata, bucketing for CUDA-graph replay and the
device-side token feedback table used when the host runs one step ahead."""
import torch

from unillm_b200.engine.runner import StepBatch, StepPacker


def _packer(max_blocks=8):
    buf = torch.zeros(1 << 14, dtype=torch.int32)
    return StepPacker(buf, max_blocks), buf


def _batch():
    # 3 decode rows, then prefill chunks of 5 and 2 tokens; the first chunk finishes its prompt (sampled)
    toks = [11, 12, 13] + [21, 22, 23, 24, 25] + [31, 32]
    pos = [40, 41, 42] + list(range(5)) + [7, 8]
    slots = [100, 101, 102] + list(range(200, 205)) + [300, 301]
    lens = [41, 42, 43, 5, 9]
    tables = [[1, 2, 3], [4, 5, 6], [7, 8, 9], [10], [11]]
    return StepBatch(toks, pos, slots, 3, lens, tables, [5, 2], [0, 1, 2, 7])


def test_pack_plain_layout():
    pk, buf = _packer()
    lay = pk.pack(_batch(), bucketed=False)
    def view(name):
        o, n = lay[name]
        return buf[o:o + n].tolist()

    assert view("token_ids") == [11, 12, 13, 21, 22, 23, 24, 25, 31, 32]
    assert view("seq_lens_d") == [41, 42, 43] and view("seq_lens_p") == [5, 9]
    assert view("q_start") == [0, 5, 7]
    assert view("sample_rows") == [0, 1, 2, 7] and lay["_sel"] == [0, 1, 2, 3]
    bt = torch.tensor(view("block_tables")).view(5, 8)
    assert bt[1, :3].tolist() == [4, 5, 6] and bt[3, 0].item() == 10
    assert (lay["_T"], lay["_D"], lay["_Dp"], lay["_P"], lay["_S"], lay["_max_q"]) == (10, 3, 3, 2, 4, 5)
    assert "token_src" not in lay
    assert all(o % 4 == 0 for k, v in lay.items() if isinstance(v, tuple) for o in [v[0]])    # 16-byte aligned arrays


def test_pack_bucketed_and_token_feedback():
    pk, buf = _packer()
    lay = pk.pack(_batch(), bucketed=True, token_src=[5, -1, 2])
    def view(name):
        o, n = lay[name]
        return buf[o:o + n].tolist()

    # decode rows padded to 4, prefill tokens padded to 128 with a dummy sequence, prefill sequences to a power of two
    assert lay["_Dp"] == 4 and lay["_T"] == 4 + 128 and lay["_P"] == 4
    assert view("token_ids")[:4] == [11, 12, 13, 0] and view("token_ids")[4:11] == [21, 22, 23, 24, 25, 31, 32]
    assert view("slot_mapping")[3] == -1 and view("slot_mapping")[4 + 7] == -1          # padding writes no KV
    assert view("seq_lens_d") == [41, 42, 43, 1]
    assert view("token_src") == [5, -1, 2, -1]
    assert view("q_start") == [0, 5, 7, 128, 128]
    # every decode row and the last row of every prefill sequence is sampled; _sel picks the requested ones
    rows = view("sample_rows")
    assert rows[:4] == [0, 1, 2, 3] and rows[4] == 4 + 4 and rows[5] == 4 + 6
    assert lay["_sel"] == [0, 1, 2, 4]
    assert lay["_max_q"] == 128
