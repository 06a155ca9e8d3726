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
