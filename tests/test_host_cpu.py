"""Host-side logic that needs no GPU: pack/unpack glue, mask analysis, model patch wiring, sharding (gloo, 2 ranks)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_pad_unpad_round_trip():
    from turbodeberta_b200 import padding
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 7, 2, 4, generator=g)
    mask = torch.tensor([[1, 1, 1, 0, 0, 0, 0], [1, 1, 1, 1, 1, 1, 1], [0, 1, 0, 1, 1, 0, 0]])
    toks, idx, cu, mx = padding.unpad_input(x, mask)
    assert toks.shape == (13, 2, 4) and cu.tolist() == [0, 3, 10, 13] and mx == 7 and cu.dtype == torch.int32
    assert torch.equal(toks, x.reshape(21, 2, 4)[mask.flatten().bool()])
    back = padding.pad_input(toks, idx, 3, 7)
    assert torch.equal(back, x * mask[:, :, None, None])
    q, k, v, pk, pq, iq, (cq, ck), (mq, mk) = padding._upad_input(x, x + 1, x + 2, "kr", "qr", mask, 7, 2)
    assert torch.equal(k, toks + 1) and torch.equal(v, toks + 2) and pk == "kr" and pq == "qr"
    assert torch.equal(cq, cu) and mq == mk == 7 and torch.equal(iq, idx)
    with pytest.raises(NotImplementedError):
        padding._upad_input(x[:, :1], x, x, None, None, mask, 1, 2)


def test_mask_analysis():
    from turbodeberta_b200.model import analyse_mask

    def ext(m):
        e = m[:, None, None, :]
        return e * e.squeeze(-2).unsqueeze(-1)

    i = analyse_mask(ext(torch.ones(2, 5)), 2, 5)
    assert i.all_ones and i.right_padded
    i = analyse_mask(ext(torch.tensor([[1, 1, 0, 0, 0], [1, 1, 1, 1, 1]])), 2, 5)
    assert not i.all_ones and i.right_padded and i.seqlens.tolist() == [2, 5]
    i = analyse_mask(torch.tensor([[0, 0, 1, 1, 1], [1, 1, 1, 1, 1]]), 2, 5)
    assert not i.right_padded and i.seqlens.tolist() == [3, 5]
    with pytest.raises(ValueError):
        analyse_mask(torch.tril(torch.ones(1, 1, 5, 5)), 1, 5)
    assert analyse_mask(None, 1, 5).all_ones


def test_patch_classes_keep_hf_parameter_names():
    from transformers import DebertaV2Config
    from transformers.models.deberta_v2.modeling_deberta_v2 import DebertaV2Model
    from turbodeberta_b200 import model as M
    cfg = DebertaV2Config(vocab_size=300, hidden_size=128, num_hidden_layers=2, num_attention_heads=2,
                          intermediate_size=256, relative_attention=True, position_buckets=256,
                          max_relative_positions=-1, norm_rel_ebd="layer_norm", share_att_key=True,
                          pos_att_type=["p2c", "c2p"], position_biased_input=False, type_vocab_size=0)
    hf = DebertaV2Model(cfg)
    fl = M.FlashDebertaV2Model(cfg)
    assert list(fl.state_dict()) == list(hf.state_dict())
    fl.load_state_dict(hf.state_dict())
    assert all(isinstance(l.attention.self, M.FlashDisentangledSelfAttention) for l in fl.encoder.layer)
    for cls in (M.FlashDebertaV2ForMaskedLM, M.FlashDebertaV2ForSequenceClassification,
                M.FlashDebertaV2ForTokenClassification, M.FlashDebertaV2ForQuestionAnswering,
                M.FlashDebertaV2ForMultipleChoice):
        assert isinstance(cls(cfg).deberta.encoder, M.FlashDebertaV2Encoder)
    patched = M.patch_model(DebertaV2Model(cfg))
    assert isinstance(patched.encoder, M.FlashDebertaV2Encoder)
    assert all(isinstance(l.attention.self, M.FlashDisentangledSelfAttention) for l in patched.encoder.layer)
    # eval-mode relative embeddings are computed once and stamped
    patched.eval()
    with torch.no_grad():
        a, b = patched.encoder.get_rel_embedding(), patched.encoder.get_rel_embedding()
    assert a is b and hasattr(a, "_tdb_stamp")


def test_shard_planner():
    from turbodeberta_b200 import sharding
    sl = [sharding.shard_batch(10, 4, r) for r in range(4)]
    assert [s.stop - s.start for s in sl] == [3, 3, 2, 2] and sl[0].start == 0 and sl[-1].stop == 10
    lengths = [1000, 10, 20, 900, 30, 500, 480, 40]
    plan = sharding.shard_packed(lengths, 2)
    assert sorted(sum(plan, [])) == list(range(8))
    cost = [sum(lengths[i] ** 2 for i in p) for p in plan]
    assert max(cost) / min(cost) < 1.35


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _gather_worker(rank, world, port, ret):
    from turbodeberta_b200 import sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(5 * 3 * 2, dtype=torch.float32).view(5, 3, 2)
        sl = sharding.shard_batch(5, world, rank)
        got = sharding.gather_padded(full[sl] * 1.0, 5)
        ok1 = torch.equal(got, full)
        lengths = [4, 1, 7, 2, 5]
        plan = sharding.shard_packed(lengths, world)
        cu = np.concatenate([[0], np.cumsum(lengths)])
        stream = torch.arange(int(cu[-1]) * 2, dtype=torch.float32).view(-1, 2)
        local = torch.cat([stream[cu[s]:cu[s + 1]] for s in plan[rank]], 0) if plan[rank] else stream[:0]
        got2 = sharding.gather_packed(local, lengths, plan)
        ok2 = torch.equal(got2, stream)
        ret[rank] = bool(ok1 and ok2)
    finally:
        dist.destroy_process_group()


def test_gather_two_ranks_gloo():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    mp.spawn(_gather_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_reference_import_paths_resolve_to_this_package():
    """Code written against the reference imports ``turbodeberta.*`` (``src/turbodeberta/`` there): the alias package
    serves the same module paths and names from this implementation."""
    import turbodeberta.model as m
    import turbodeberta.ops.flash_attention as fa
    import turbodeberta.ops.flash_attention_varlen as fav
    import turbodeberta.padding as pad
    import turbodeberta_b200.model as ours
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    from turbodeberta_b200.ops.flash_attention_varlen import flash_attention_with_disentangled_varlen
    assert m.FlashDebertaV2Model is ours.FlashDebertaV2Model
    assert m.FlashDisentangledSelfAttention is ours.FlashDisentangledSelfAttention
    for name in ("FlashDebertaV2Attention", "FlashDebertaV2Layer", "FlashDebertaV2Encoder", "FlashDebertaV2ForMaskedLM",
                 "FlashDebertaV2ForSequenceClassification", "FlashDebertaV2ForTokenClassification",
                 "FlashDebertaV2ForQuestionAnswering", "FlashDebertaV2ForMultipleChoice"):
        assert getattr(m, name) is getattr(ours, name)
    assert fa.flash_attention_with_disentangled is flash_attention_with_disentangled
    assert fav.flash_attention_with_disentangled_varlen is flash_attention_with_disentangled_varlen
    for name in ("pad_input", "unpad_input", "_upad_input", "index_first_axis", "index_put_first_axis", "_get_unpad_data"):
        assert callable(getattr(pad, name))


def test_pending_status_blocks_are_folded_never_dropped():
    """Unchecked status blocks pile up only to a bound, and a report in the very first one survives the folding."""
    from turbodeberta_b200.status import PendingStatus
    q = PendingStatus()
    first = torch.tensor([7, 0, 0, 0], dtype=torch.int32)
    q.append(first)
    for _ in range(3 * PendingStatus.FOLD_AT):
        q.append(torch.zeros(4, dtype=torch.int32))
    assert len(q) < PendingStatus.FOLD_AT
    blocks = q.drain()
    assert len(q) == 0
    assert int(torch.stack(blocks).amax(dim=0)[0]) == 7


def test_mask_analysis_refresh_recomputes_lengths_without_changing_the_route():
    from turbodeberta_b200.model import analyse_mask
    m = torch.zeros(2, 6, dtype=torch.long)
    m[0, :6] = 1
    m[1, :3] = 1
    a = analyse_mask(m, 2, 6)
    assert (a.all_ones, a.right_padded) == (False, True) and a.seqlens.tolist() == [6, 3]
    b = analyse_mask(m, 2, 6, refresh=True)
    assert b is not a and (b.all_ones, b.right_padded) == (False, True) and b.seqlens.tolist() == [6, 3]
    assert analyse_mask(m, 2, 6) is b                      # the refreshed analysis is what later calls see
