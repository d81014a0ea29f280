"""Speech input: token count formula, the Whisper tower against Hugging Face's WhisperEncoder, the audio server's
manager over an in-process embed cache."""
import numpy as np
import torch


def test_audio_token_counts():
    from lightllm_b200.models.whisper_audio import audio_token_num, chunk_lengths, frames_after_cnn

    assert frames_after_cnn(3000) == 1500 and frames_after_cnn(3) == 2
    assert audio_token_num(480000) == 750          # 30 s -> 1500 frames -> 750 embeddings (one per 40 ms)
    assert audio_token_num(16000) == 25            # 1 s -> 100 mel frames -> 50 -> 25
    assert chunk_lengths(480000 + 16000) == [480000, 16000] and audio_token_num(480000 + 16000) == 775
    assert audio_token_num(100) == audio_token_num(480)   # short clips are padded to 480 samples


def _tiny(tmp=None):
    from transformers import WhisperConfig, WhisperModel

    torch.manual_seed(0)
    wc = WhisperConfig(d_model=32, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=64, num_mel_bins=80,
                       max_source_positions=1500, decoder_layers=1, decoder_attention_heads=4, decoder_ffn_dim=64,
                       vocab_size=100, pad_token_id=0, bos_token_id=1, eos_token_id=2, decoder_start_token_id=1)
    enc = WhisperModel(wc).encoder.eval().float()
    sd = {"audio_model.encoder." + k: v.detach().clone() for k, v in enc.state_dict().items()}
    g = torch.Generator().manual_seed(1)
    sd.update({"mlp2.0.weight": torch.ones(32), "mlp2.0.bias": torch.zeros(32),
               "mlp2.1.weight": torch.randn(48, 32, generator=g) * 0.1, "mlp2.1.bias": torch.zeros(48),
               "mlp2.3.weight": torch.randn(48, 48, generator=g) * 0.1, "mlp2.3.bias": torch.zeros(48)})
    cfg = {"model_type": "internvl_chat", "llm_config": {"hidden_size": 48},
           "audio_config": {"d_model": 32, "encoder_layers": 2, "encoder_attention_heads": 4, "encoder_ffn_dim": 64,
                            "num_mel_bins": 80, "max_source_positions": 1500}}

    class Src:
        def has(self, n):
            return n in sd

        def get(self, n, *a):
            return sd[n]

        def names(self):
            return list(sd)

    return enc, cfg, Src()


def test_whisper_tower_matches_hf_encoder():
    from lightllm_b200.models.whisper_audio import WhisperAudioTower, audio_token_num

    enc, cfg, src = _tiny()
    tower = WhisperAudioTower(cfg, src, torch.device("cpu"), torch.float32)
    assert set(WhisperAudioTower.weight_shapes(cfg)) == set(src.names())
    rng = np.random.default_rng(0)
    audio = (rng.standard_normal(480000) * 0.1).astype(np.float32)       # a full 30 s window
    mel = tower.log_mel(audio)
    assert mel.shape == (80, 3000)
    with torch.no_grad():
        want = enc(mel.unsqueeze(0)).last_hidden_state[0]
    got = tower.encode_features(mel, pool=False)
    assert (got - want).abs().max().item() < 1e-4
    short = (rng.standard_normal(16000 * 3 + 77) * 0.1).astype(np.float32)
    emb = tower.encode_audio(short)
    assert emb.shape == (audio_token_num(short.shape[0]), 48) and torch.isfinite(emb).all()
    long = np.concatenate([audio, short])
    assert tower.encode_audio(long).shape[0] == audio_token_num(long.shape[0]) == 750 + emb.shape[0]


def test_audio_manager_embeds_pending_clips():
    from lightllm_b200.models.whisper_audio import WhisperAudioTower, audio_token_num
    from lightllm_b200.server.audioserver.manager import AudioManager
    from lightllm_b200.server.core.objs.io_objs import GroupReqIndexes

    _, cfg, src = _tiny()
    tower = WhisperAudioTower(cfg, src, torch.device("cpu"), torch.float32)
    clip = (np.random.default_rng(2).standard_normal(20000) * 0.1).astype(np.float32)
    n = audio_token_num(clip.shape[0])

    class Arena:
        def __init__(self):
            self.rows = {}

        def write(self, start, e):
            self.rows[start] = e.clone()

    class Cache:
        def __init__(self):
            self.arena, self.ready = Arena(), set()

        def get_items_embed(self, ids):
            return [i in self.ready for i in ids]

        def get_payload(self, uid):
            return clip.tobytes()

        def set_items_embed(self, ids):
            self.ready.update(ids)

    cache, sent = Cache(), []
    mgr = AudioManager(None, tower, cache, sent.append, None)
    item = {"uuid": 7, "token_id": 100_000_000, "token_num": n, "start_index_in_embed_cache": 5}
    g = GroupReqIndexes.__new__(GroupReqIndexes)
    g.multimodal_params = {"images": [], "audios": [item]}
    mgr.handle(g)
    assert sent == [g] and 7 in cache.ready and cache.arena.rows[5].shape == (n, 48)
    mgr.handle(g)   # already embedded: passes straight through
    assert len(sent) == 2


def test_qwen3_omni_tokenizer_expands_audio_and_image_placeholders():
    from types import SimpleNamespace

    from lightllm_b200.models.qwen3_omni import Qwen3OmniTokenizer, audio_token_num

    class Tok:
        def encode(self, text, add_special_tokens=False):
            return [int(x) for x in text.split()]

    cfg = {"image_token_id": 290, "audio_token_id": 288, "vision_config": {"patch_size": 16, "spatial_merge_size": 2},
           "audio_config": {"n_window": 50}}
    tk = Qwen3OmniTokenizer(Tok(), cfg)
    clip = SimpleNamespace(audio_length=16000 * 3 + 700, token_id=5000, token_num=0)
    clip.token_num = tk.get_audio_token_length(clip)
    assert clip.token_num == audio_token_num(48700) == 3 * 13 + 1        # 304 frames: three windows and 4 frames
    img = SimpleNamespace(token_id=7000, token_num=6)
    mp = SimpleNamespace(images=[img], audios=[clip])
    ids = tk.encode("1 292 290 293 2 294 288 295 3", mp)
    assert ids == [1, 292] + list(range(7000, 7006)) + [293, 2, 294] + list(range(5000, 5000 + clip.token_num)) + [295, 3]
    import pytest

    with pytest.raises(ValueError):
        tk.encode("1 294 295", mp)
