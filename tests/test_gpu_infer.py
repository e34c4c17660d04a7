"""Forward-only use of the attention kernel: the reference's inference attention module, its
Hugging Face attention module and its perplexity scorer (all of which call SDPA in the reference)
with the kernel patched in, against their oracle restatements."""
import numpy as np
import pytest
import torch

from oracle import infer as oinfer, model as omodel, ops
from tests.golden import inputs

pytestmark = pytest.mark.gpu


def _tables(d_model, L):
    cos, sin = ops.rope_tables(d_model, L)
    return cos.cuda().unsqueeze(0), sin.cuda().unsqueeze(0)      # [1, L, d_model] like the models' buffers


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_patched_inference_attention_matches_its_sdpa_forward(dtype):
    import ulm_infer
    torch.manual_seed(0)
    d, H, L = 256, 4, 300
    attn = oinfer.InfAttention(d, H).cuda()
    x = torch.randn(3, L, d, device='cuda')
    cos, sin = _tables(d, L)
    with torch.no_grad(), torch.autocast('cuda', dtype=dtype):
        want = attn(x, cos=cos, sin=sin)
        assert ulm_infer.patch_attention(attn) == 1
        got = attn(x, cos=cos, sin=sin)
        # what the kernel does not cover goes to the module's own code: a mask, or autograd being on
        masked = attn(x, mask=torch.ones(L, L, dtype=torch.bool, device='cuda').tril(), cos=cos, sin=sin)
    with torch.autocast('cuda', dtype=dtype):
        with_grad = attn(x, cos=cos, sin=sin)
    ulm_infer.unpatch_attention(attn)
    tol = 2e-3 if dtype == torch.float16 else 1e-2
    assert float((got.float() - want.float()).norm() / want.float().norm()) < tol
    assert float((masked.float() - want.float()).norm() / want.float().norm()) < tol
    assert with_grad.requires_grad
    import flash_attn_v100_cuda as fa
    fa.check_status()


def test_patched_hf_attention_prefill_returns_the_same_cache_and_decodes_on():
    import ulm_infer
    torch.manual_seed(1)
    d, H, L = 128, 2, 70
    dtype = torch.float16
    attn = oinfer.HFAttention(d, H, layer_idx=0).cuda().to(dtype)
    x = torch.randn(2, L + 1, d, device='cuda', dtype=dtype)
    cos, sin = _tables(d, L + 1)
    with torch.no_grad():
        want, (k0, v0) = attn(x[:, :L], cos[:, :L], sin[:, :L], use_cache=True)
        assert ulm_infer.patch_attention(attn) == 1
        got, (k1, v1) = attn(x[:, :L], cos[:, :L], sin[:, :L], use_cache=True)          # prefill through the kernel
        assert torch.equal(k1, k0.to(dtype)) and torch.equal(v1, v0)                     # same cache, bit for bit
        # one cached decode step: not the kernel's case, goes to the module's own forward, on our cache
        step_want, _ = attn._ulm_original_forward(x[:, L:], cos[:, L:], sin[:, L:], past_key_value=(k0, v0), is_causal=False)
        step_got, _ = attn(x[:, L:], cos[:, L:], sin[:, L:], past_key_value=(k1, v1), is_causal=False)
    assert float((got.float() - want.float()).norm() / want.float().norm()) < 2e-3
    assert torch.equal(step_got, step_want)


def test_model_logits_and_scoring_match_the_sdpa_path():
    """Last-token logits at the thresholds the reference's own export check uses for half precision
    (convert_to_hf.py:451-455: max |delta| <= 1.5e-1; here also 2e-2) and the perplexity scorer's
    per-window sums (inf.py:866-937)."""
    import ulm_infer
    import ulm_model
    cfg = dict(vocab_size=4096, d_model=128, n_heads=2, n_layers=2, d_ff=344, max_seq_len=256)
    prod = ulm_model.DecoderOnlyTransformer(ulm_model.ModelConfig(**cfg)).cuda().eval()
    prod.load_state_dict(inputs.seeded_weights(0, cfg), strict=False)
    orc = omodel.OracleLM(omodel.OracleModelConfig(**cfg))
    inputs.load_seeded_weights_into_oracle(orc)
    orc = orc.cuda().eval()
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(3, 4096, (2, 32), generator=g).cuda()
    with torch.no_grad(), torch.autocast('cuda', dtype=torch.float16):
        got = prod(ids)[:, -1].float()
        want = orc.fc_out(orc.hidden(ids))[:, -1].float()
    diff = (got - want).abs()
    assert float(diff.max()) <= 2e-2 and float(diff.max()) <= 1.5e-1
    assert float(torch.nn.functional.cosine_similarity(got, want).min()) > 0.9999
    rng = np.random.default_rng(5)
    windows = [rng.integers(3, 4096, size=int(n)).tolist() for n in (2, 17, 64, 200, 257, 33, 1, 129)]
    dev = torch.device('cuda')
    l1, t1, c1 = ulm_infer.score_windows(prod, windows, 0, dev, batch_size=3, chunk_rows=100)
    l2, t2, c2 = oinfer.score_windows(orc, windows, 0, dev, batch_size=3, chunk_rows=100)
    assert t1 == t2
    for a, b, n in zip(l1, l2, t1):
        assert abs(a - b) <= 2e-3 * max(1, n), (a, b, n)
    assert all(abs(a - b) <= 1 for a, b in zip(c1, c2))           # an argmax tie may fall either way
