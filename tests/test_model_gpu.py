"""GPU parity of the patched HF modules against the eager modules they replace."""
import numpy as np
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu


def _cfg(**kw):
    from transformers import DebertaV2Config
    base = dict(vocab_size=500, hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=256,
                relative_attention=True, position_buckets=256, max_relative_positions=-1, norm_rel_ebd="layer_norm",
                share_att_key=True, pos_att_type=["p2c", "c2p"], position_biased_input=False, type_vocab_size=0,
                hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    base.update(kw)
    return DebertaV2Config(**base)


def _ext(mask2d):
    e = mask2d[:, None, None, :]
    return e * e.squeeze(-2).unsqueeze(-1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mask_kind", ["ones", "right", "left"])
@pytest.mark.parametrize("share,pos", [(True, ["c2p", "p2c"]), (False, ["c2p", "p2c"]), (True, ["c2p"]), (True, [])])
def test_attention_module_matches_eager(dtype, mask_kind, share, pos):
    from transformers.models.deberta_v2.modeling_deberta_v2 import DisentangledSelfAttention
    from turbodeberta_b200.model import FlashDisentangledSelfAttention
    torch.manual_seed(3)
    cfg = _cfg(share_att_key=share, pos_att_type=pos, relative_attention=len(pos) > 0)
    ref = DisentangledSelfAttention(cfg).eval()
    with torch.no_grad():
        for p in ref.parameters():
            p.normal_(0, 0.05)
    B, L = 3, 200
    x = torch.randn(B, L, 128)
    rel = torch.randn(512, 128) * 0.1
    lens = {"ones": [L, L, L], "right": [200, 37, 129], "left": [200, 37, 129]}[mask_kind]
    m = torch.zeros(B, L, dtype=torch.long)
    for b, n in enumerate(lens):
        if mask_kind == "left":
            m[b, L - n:] = 1
        else:
            m[b, :n] = 1
    # reference: fp32 eager on the same (dtype-rounded) parameters and inputs
    ref_r = DisentangledSelfAttention(cfg).eval()
    ref_r.load_state_dict({k: v.to(dtype).float() for k, v in ref.state_dict().items()})
    xr, relr = x.to(dtype).float(), rel.to(dtype).float()
    with torch.no_grad():
        want, _ = ref_r(xr, _ext(m).bool(), relative_pos=None, rel_embeddings=relr)
    fl = FlashDisentangledSelfAttention(cfg).eval()
    fl.load_state_dict(ref.state_dict())
    fl = fl.to("cuda", dtype)
    with torch.no_grad():
        got, probs = fl(x.to("cuda", dtype), _ext(m).to("cuda"), rel_embeddings=rel.to("cuda", dtype))
    assert probs is None and got.shape == (B, L, 128)
    valid = m.bool()
    g, w = got.float().cpu()[valid].numpy(), want[valid].numpy()
    if dtype == torch.float32:
        assert np.abs(g - w).max() / np.abs(w).max() < util.FP32_REL_TOL
    else:
        # Q/K/V are rounded to bf16 after the projection in the fused path only; allow for it on top of the kernel tolerance
        assert np.abs(g - w).max() < 2 * util.BF16_ABS_TOL
    assert torch.count_nonzero(got.float().cpu()[~valid]).item() == 0


def test_whole_model_matches_eager_fp32():
    from transformers.models.deberta_v2.modeling_deberta_v2 import DebertaV2Model
    from turbodeberta_b200.model import FlashDebertaV2Model, patch_model
    torch.manual_seed(5)
    cfg = _cfg()
    hf = DebertaV2Model(cfg).eval()
    fl = FlashDebertaV2Model(cfg).eval()
    fl.load_state_dict(hf.state_dict())
    ids = torch.randint(0, 500, (3, 160))
    mask = torch.ones(3, 160, dtype=torch.long)
    mask[1, 100:] = 0
    mask[2, 33:] = 0
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask).last_hidden_state
        got = fl.cuda()(input_ids=ids.cuda(), attention_mask=mask.cuda()).last_hidden_state.cpu()
        got2 = fl(input_ids=ids.cuda(), attention_mask=mask.cuda()).last_hidden_state.cpu()      # cached tables
    v = mask.bool()
    assert (got[v] - want[v]).abs().max().item() / want[v].abs().max().item() < 2e-4
    assert torch.equal(got, got2)
    patched = patch_model(DebertaV2Model(cfg).eval())
    patched.load_state_dict(hf.state_dict())
    with torch.no_grad():
        got3 = patched.cuda()(input_ids=ids.cuda(), attention_mask=mask.cuda()).last_hidden_state.cpu()
    assert (got3[v] - want[v]).abs().max().item() / want[v].abs().max().item() < 2e-4


def test_tables_follow_weight_updates():
    """The cached relative tables must be rebuilt when a projection weight changes in place."""
    from turbodeberta_b200.model import FlashDebertaV2Model
    torch.manual_seed(6)
    fl = FlashDebertaV2Model(_cfg()).eval().cuda()
    ids = torch.randint(0, 500, (1, 64)).cuda()
    with torch.no_grad():
        a = fl(input_ids=ids).last_hidden_state.clone()
        fl.encoder.layer[0].attention.self.key_proj.weight.mul_(1.5)
        b = fl(input_ids=ids).last_hidden_state
    assert not torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_packed_encoder_route_matches_padded_route(dtype):
    """Padded batches run on the packed token stream by default; both routes and the eager model must agree on
    every valid token, for the last layer and for the intermediate hidden states."""
    from transformers.models.deberta_v2.modeling_deberta_v2 import DebertaV2Model
    from turbodeberta_b200.model import FlashDebertaV2Model
    torch.manual_seed(8)
    cfg = _cfg(num_hidden_layers=3)
    hf = DebertaV2Model(cfg).eval()
    fl = FlashDebertaV2Model(cfg).eval()
    fl.load_state_dict(hf.state_dict())
    fl = fl.to("cuda", dtype)
    ids = torch.randint(0, 500, (4, 300))
    mask = torch.zeros(4, 300, dtype=torch.long)
    for b, n in enumerate([300, 17, 129, 256]):
        mask[b, :n] = 1
    v = mask.bool()
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask, output_hidden_states=True)
        assert fl.encoder.pack_padded_batches
        packed = fl(input_ids=ids.cuda(), attention_mask=mask.cuda(), output_hidden_states=True)
        fl.encoder.pack_padded_batches = False
        padded = fl(input_ids=ids.cuda(), attention_mask=mask.cuda(), output_hidden_states=True)
        fl.encoder.pack_padded_batches = True
    assert len(packed.hidden_states) == len(want.hidden_states) == 4
    tol = 2e-4 if dtype == torch.float32 else 6e-2
    for a, b_, c in zip(packed.hidden_states, padded.hidden_states, want.hidden_states):
        a, b_ = a.float().cpu(), b_.float().cpu()
        scale = c[v].abs().max().item()
        assert (a[v] - c[v]).abs().max().item() / scale < tol
        assert (a[v] - b_[v]).abs().max().item() / scale < tol
    assert torch.count_nonzero(packed.last_hidden_state.float().cpu()[~v]).item() == 0
    assert torch.equal(packed.last_hidden_state, packed.hidden_states[-1])


def test_encoder_forward_captures_into_a_cuda_graph():
    """After a warm-up with the same mask tensor (tables, fused weights and the mask analysis are cached) the whole
    model forward records into a CUDA graph: no allocation in the library, no synchronisation on the path; the
    replay reproduces the eager forward bit for bit and leaves the status words for the next check."""
    from turbodeberta_b200.model import FlashDebertaV2Model
    from turbodeberta_b200.ops.flash_attention import check_pending_status
    torch.manual_seed(9)
    model = FlashDebertaV2Model(_cfg(num_hidden_layers=3)).eval().cuda().to(torch.bfloat16)
    ids = torch.randint(0, 500, (4, 256), device="cuda")
    mask = torch.ones_like(ids)

    @torch.no_grad()
    def fwd():
        return model(input_ids=ids, attention_mask=mask).last_hidden_state

    eager = fwd().clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fwd()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = fwd()
    ids.copy_(torch.randint(0, 500, (4, 256), device="cuda"))        # new contents in the captured input buffer
    graph.replay()
    torch.cuda.synchronize()
    check_pending_status()                                           # the replay's status words are readable now
    fresh = fwd()
    assert torch.equal(out, fresh)
    assert not torch.equal(out, eager)


def _config4():
    """Configuration 4's model: DeBERTa-v3-large geometry, random init."""
    from transformers import DebertaV2Config
    return DebertaV2Config(vocab_size=128100, hidden_size=1024, num_hidden_layers=24, num_attention_heads=16,
                           intermediate_size=4096, hidden_act="gelu", relative_attention=True, position_buckets=256,
                           max_relative_positions=-1, max_position_embeddings=512, norm_rel_ebd="layer_norm",
                           share_att_key=True, pos_att_type=["p2c", "c2p"], position_biased_input=False, type_vocab_size=0)


def test_config4_model_at_full_size_matches_eager():
    """The 24-layer, hidden-1024, 16-head model of configuration 4 on 512-token sequences against the eager model in
    fp32 on the host: bf16 on 2 x 512 tokens (tensor-core kernel), fp32 on 1 x 512 tokens (exact kernel)."""
    from transformers.models.deberta_v2.modeling_deberta_v2 import DebertaV2Model
    from turbodeberta_b200.model import FlashDebertaV2Model
    torch.manual_seed(1004)
    cfg = _config4()
    hf = DebertaV2Model(cfg).eval()
    sd_bf = {k: v.to(torch.bfloat16) for k, v in hf.state_dict().items()}
    hf.load_state_dict({k: v.float() for k, v in sd_bf.items()})          # fp32 model holding the bf16-rounded weights
    gen = torch.Generator().manual_seed(1004)
    ids = torch.randint(0, 128100, (2, 512), generator=gen)
    mask = torch.ones_like(ids)
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask).last_hidden_state
    fl = FlashDebertaV2Model(cfg).eval()
    fl.load_state_dict(hf.state_dict())
    # fp32, one sequence
    fl32 = fl.to("cuda")
    with torch.no_grad():
        got32 = fl32(input_ids=ids[:1].cuda(), attention_mask=mask[:1].cuda()).last_hidden_state.cpu()
    rel = (got32 - want[:1]).abs().max().item() / want[:1].abs().max().item()
    assert rel < util.MODEL_FP32_REL_TOL, rel
    # bf16, both sequences; yardstick: the eager model in bf16 on the same GPU
    flbf = fl32.to(torch.bfloat16)
    with torch.no_grad():
        got = flbf(input_ids=ids.cuda(), attention_mask=mask.cuda()).last_hidden_state.float().cpu()
    del flbf, fl32, fl
    eager_bf = DebertaV2Model(cfg).eval()
    eager_bf.load_state_dict(hf.state_dict())
    eager_bf = eager_bf.to("cuda", torch.bfloat16)
    with torch.no_grad():
        eag = eager_bf(input_ids=ids.cuda(), attention_mask=mask.cuda()).last_hidden_state.float().cpu()
    del eager_bf
    torch.cuda.empty_cache()
    assert torch.isfinite(got).all()
    err_ours, err_eager = (got - want).abs(), (eag - want).abs()
    f = util.MODEL_BF16_VS_EAGER_FACTOR
    assert err_ours.max().item() <= f * err_eager.max().item(), (err_ours.max().item(), err_eager.max().item())
    assert err_ours.pow(2).mean().sqrt().item() <= f * err_eager.pow(2).mean().sqrt().item()


def test_task_head_classes_run_on_the_gpu():
    """The five head classes (broken constructors upstream, ``model.py:244-314``) through the fused kernels against
    their eager counterparts with the same weights, fp32, padded batch."""
    import transformers.models.deberta_v2.modeling_deberta_v2 as hfm
    import turbodeberta_b200.model as ours
    torch.manual_seed(11)
    cfg = _cfg(num_labels=2)                 # the question-answering head splits its output in two
    ids = torch.randint(0, 500, (3, 96))
    mask = torch.ones_like(ids)
    mask[1, 50:] = 0
    for name in ("ForMaskedLM", "ForSequenceClassification", "ForTokenClassification", "ForQuestionAnswering",
                 "ForMultipleChoice"):
        hf = getattr(hfm, "DebertaV2" + name)(cfg).eval()
        fl = getattr(ours, "FlashDebertaV2" + name)(cfg).eval()
        fl.load_state_dict(hf.state_dict())
        x, m = (ids[None], mask[None]) if name == "ForMultipleChoice" else (ids, mask)       # [1, choices, L]
        with torch.no_grad():
            want = hf(input_ids=x, attention_mask=m)
            got = fl.cuda()(input_ids=x.cuda(), attention_mask=m.cuda())
        outs = [("start_logits", "end_logits")] if name == "ForQuestionAnswering" else [("logits",)]
        for fields in outs:
            for f in fields:
                a, b = getattr(got, f).float().cpu(), getattr(want, f)
                if name in ("ForMaskedLM", "ForTokenClassification", "ForQuestionAnswering"):       # per-token outputs
                    v = mask.bool()
                    a, b = a[v], b[v]
                assert (a - b).abs().max().item() / max(b.abs().max().item(), 1e-6) < 5e-4, (name, f)
        del hf, fl
