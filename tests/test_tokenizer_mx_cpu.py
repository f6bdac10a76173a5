"""Tokenizer files / extended vocabulary and the MX (block-scaled fp8) reference arithmetic, on CPU."""
import torch

from pisceslx_b200.models.tokenizer import YvExtendedTokenizerConfig, YvTokenizer, YvTokenizer160K, train_tokenizer


def test_shipped_tokenizer_round_trips_and_keeps_special_ids():
    YvTokenizer.reset_instance()
    tok = YvTokenizer.instance()
    assert tok.backend is not None and tok.vocab_size == 8192            # the file under tokenizer/
    assert (tok.pad_token_id, tok.bos_token_id, tok.eos_token_id) == (0, 1, 2)
    s = "def f(x):\n    return x * 2  # ünïcødé 中文 <think>ok</think>"
    ids = tok.encode(s, add_bos=True, add_eos=True)
    assert ids[0] == 1 and ids[-1] == 2 and tok.decode(ids[1:-1], skip_special_tokens=False) == s
    assert tok.get_special_token_id("<think>") in ids and len(ids) < len(s.encode())
    assert tok.batch_decode(tok.encode_batch(["ab", "cd"])) == ["ab", "cd"]
    assert tok.convert_ids_to_tokens([tok.im_start_id]) == ["<|im_start|>"]
    small = YvTokenizer.for_vocab(512)                                    # model too small for the file: byte ids
    assert small.backend is None and max(small.encode("hello")) < 512
    assert YvTokenizer.for_vocab(154856) is tok


def test_train_tokenizer_and_save_pretrained(tmp_path):
    corpus = tmp_path / "c.txt"
    corpus.write_text("the quick brown fox jumps over the lazy dog\n" * 50 + "pack my box with five dozen liquor jugs\n" * 50)
    out = train_tokenizer([corpus], tmp_path / "tok", vocab_size=400)
    t = YvTokenizer(out)
    assert t.backend is not None and 280 < t.vocab_size <= 400
    assert t.decode(t.encode("the quick fox ∑")) == "the quick fox ∑"            # bytes outside the corpus survive
    n = t.add_tokens(["<new_a>", "<new_b>", "<|pad|>"])
    assert n == 2 and t.decode([t.get_special_token_id("<new_a>")], skip_special_tokens=False) == "<new_a>"
    t.save_pretrained(tmp_path / "saved")
    assert YvTokenizer(tmp_path / "saved").vocab_size == t.vocab_size


def test_extended_160k_vocabulary_ranges():
    cfg = YvExtendedTokenizerConfig(target_vocab_size=12000, num_scientific_tokens=1000, num_code_tokens=800,
                                    num_multilingual_tokens=700, num_domain_tokens=500)
    e = YvTokenizer160K(cfg)
    assert e.is_extended and e.get_extended_vocab_size() == 12000 and e.base_vocab_size == 8192
    sci, code = e.get_domain_token_ids("scientific"), e.get_domain_token_ids("code")
    assert len(sci) == 1000 and len(code) == 800 and sci[-1] + 1 == code[0]
    ids = e.encode("α_3 == β^2")
    assert any(i in set(sci) for i in ids) and any(i in set(code) for i in ids)
    assert e.decode(ids) == "α_3 == β^2"
    assert len(e.get_extended_vocab()) == 12000 - 8192


def test_mx_reference_quantisation_and_chunk_layout():
    from pisceslx_b200.quant import fp8 as q8
    torch.manual_seed(0)
    x = (torch.randn(200, 256) * torch.logspace(-3, 2, 256)).bfloat16().float()
    x[0, :32] = 0
    x[1, 0], x[1, 1:32] = 448.0, 0.1
    x[2, 0], x[2, 1:32] = 449.0, 0.0
    q, e = q8.quantize_mx_reference(x)
    assert int(e[0, 0]) == 127 and int(e[1, 0]) == 127 and int(e[2, 0]) == 128      # 448 fits, 449 needs the next power
    d = q8.dequantize_mx(q, e)
    assert float((d - x).abs().max() / x.abs().max()) < 0.04
    blocks = (d - x).view(200, 8, 32).abs().amax(-1) / x.view(200, 8, 32).abs().amax(-1).clamp_min(1e-30)
    assert float(blocks.max()) < 0.07                                     # every block keeps ~4 significant bits
    c = q8.mx_scales_to_chunks(e)
    assert c.shape == (2, 2, 512) and torch.equal(q8.mx_chunks_to_scales(c, 200), e)
    r, kb = 150, 5
    assert c[r // 128, kb // 4, ((r % 128) % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4] == e[r, kb]
    assert int(c[1, 0, (127 % 32) * 16 + (127 // 32) * 4]) == 127          # rows past the end hold scale 1
    q2, c2 = q8.quantize_mx(x)                                            # CPU path of the public entry
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(c2, c)


def test_quartet_linear_stores_four_bits_and_trains_through_stochastic_rounding():
    import torch.nn as nn
    from pisceslx_b200.quant.fp4 import PiscesLxQuartetLinear, PiscesLxQuartetTrainer, pack_fp4, unpack_fp4
    torch.manual_seed(0)
    q = torch.tensor([0.0, -0.5, 6.0, -3.0, 1.5])
    assert torch.equal(unpack_fp4(pack_fp4(q), 5), q) and pack_fp4(q).numel() == 3
    lin = PiscesLxQuartetLinear(32, 16, seed=1)
    assert lin.storage_bytes() == 32 * 16 // 2 + 32 * 16 // 16 * 4           # half a byte per weight + block scales
    target = torch.randn(16, 32) * 0.02                                     # stochastic rounding is unbiased:
    acc = torch.zeros_like(target)                                          # the mean of many stores approaches the target
    for _ in range(200):
        lin.store(target)
        acc += lin.dequantized()
    one = (lin.dequantized() - target).abs().mean()
    assert float((acc / 200 - target).abs().mean()) < 0.25 * float(one)
    net = nn.Sequential(nn.Linear(8, 32), nn.ReLU(), nn.Linear(32, 1))
    tr = PiscesLxQuartetTrainer(net)
    assert tr.converted == 2 and tr.get_compression_ratio() > 3.0
    x = torch.randn(256, 8)
    y = x[:, :1] * 2 - x[:, 1:2]
    first = None
    for _ in range(300):
        loss = (net(x) - y).pow(2).mean()
        loss.backward()
        tr.step(0.05)
        first = first if first is not None else float(loss.detach())
    assert float(loss.detach()) < 0.1 * first
