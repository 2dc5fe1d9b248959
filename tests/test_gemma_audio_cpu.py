"""Gemma-4 audio tower against the Hugging Face implementation (random tiny weights loaded by name): the blocked attention with a
shifted relative-position bias of the library equals the per-query windowed form used here, across several 12-frame blocks."""
import pytest
import torch

from mary_b200.models.gemma4.audio import Gemma4AudioConfig, Gemma4AudioTower, load_into


class _DictLoader:
    def __init__(self, sd):
        self.sd = sd

    def has_weight(self, n):
        return n in self.sd

    def load_tensor(self, n, dtype):
        return self.sd[n].to(dtype)


def test_soft_tokens_match_huggingface():
    pytest.importorskip("transformers")
    from transformers.models.gemma4.configuration_gemma4 import Gemma4AudioConfig as HFA, Gemma4TextConfig
    from transformers.models.gemma4.modeling_gemma4 import Gemma4AudioModel, Gemma4MultimodalEmbedder
    c = Gemma4AudioConfig(n_mels=16, hidden=32, layers=2, heads=4, conv_channels=(16, 8), context_left=13, out_dims=24, text_hidden=20)
    torch.manual_seed(0)
    ha = HFA(hidden_size=c.hidden, num_hidden_layers=c.layers, num_attention_heads=c.heads, subsampling_conv_channels=list(c.conv_channels),
             conv_kernel_size=c.conv_kernel, attention_chunk_size=12, attention_context_left=c.context_left, attention_context_right=0,
             attention_logit_cap=c.logit_cap, output_proj_dims=c.out_dims, use_clipped_linears=True)
    ha._attn_implementation = "sdpa"          # the library builds the boolean window mask its blocked attention expects only on this path
    tower = Gemma4AudioModel(ha).eval()
    emb = Gemma4MultimodalEmbedder(ha, Gemma4TextConfig(hidden_size=c.text_hidden, num_hidden_layers=2, num_attention_heads=2,
                                                        intermediate_size=32, vocab_size=64, head_dim=8, global_head_dim=8)).eval()
    with torch.no_grad():
        for n, p in tower.named_parameters():
            if n.endswith("per_dim_scale"):
                p.copy_(0.5 * torch.randn_like(p))
            elif p.dim() == 1:
                p.copy_((0.0 if n.endswith("bias") else 1.0) + 0.1 * torch.randn_like(p))
            else:
                p.copy_(0.3 * torch.randn_like(p))
        for mod in tower.modules():
            if hasattr(mod, "input_min"):
                mod.input_min.fill_(-2.5), mod.input_max.fill_(2.5), mod.output_min.fill_(-6.0), mod.output_max.fill_(6.0)
    sd = {"model.audio_tower." + k: v.detach() for k, v in tower.state_dict().items()}
    sd.update({"model.embed_audio." + k: v.detach() for k, v in emb.state_dict().items()})
    m = Gemma4AudioTower(c)
    load_into(m, _DictLoader(sd))
    mel = torch.randn(164, c.n_mels)                                # 41 frames after subsampling: four blocks of 12, the last ragged
    with torch.no_grad():
        out = tower(mel[None], attention_mask=torch.ones(1, 164, dtype=torch.bool))
        want = emb(out.last_hidden_state)[0]
        got = m(mel)
    assert got.shape == (41, c.text_hidden)
    assert torch.allclose(got, want, atol=3e-4, rtol=3e-4), float((got - want).abs().max())
    assert m.layers[0].q.clipped


def test_log_mel_front_end_matches_the_library_feature_extractor():
    pytest.importorskip("transformers")
    import numpy as np
    from transformers.models.gemma4.feature_extraction_gemma4 import Gemma4AudioFeatureExtractor
    from mary_b200.models.gemma4.audio import usm_log_mel
    wave = (0.1 * np.random.default_rng(0).standard_normal(16000)).astype(np.float32)
    fe = Gemma4AudioFeatureExtractor()
    want = torch.as_tensor(fe([wave], sampling_rate=16000, return_tensors="pt")["input_features"][0]).float()
    got = usm_log_mel(wave)
    n = min(got.shape[0], want.shape[0])
    assert abs(got.shape[0] - want.shape[0]) <= 1 and got.shape[1] == 128
    assert torch.allclose(got[:n], want[:n], atol=1e-4), float((got[:n] - want[:n]).abs().max())
