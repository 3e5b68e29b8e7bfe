"""Weights of a Hugging Face Llama loaded into LlamaModel compute the same function: hidden
states and per-token log-probabilities agree with transformers' own forward (an independent
implementation of the architecture), on CPU."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from kernel_align_b200.models.hf_convert import config_from_hf, from_hf, to_hf_state_dict  # noqa: E402

CPU = torch.device("cpu")


def _hf_model():
    cfg = transformers.LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=128, vocab_size=512, rms_norm_eps=1e-5,
                                   rope_theta=500000.0, max_position_embeddings=256, tie_word_embeddings=False,
                                   attention_bias=False, mlp_bias=False)
    torch.manual_seed(0)
    model = transformers.LlamaForCausalLM(cfg).eval()
    # bf16-representable weights, so that both sides hold exactly the same numbers
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    return model


def test_config_mapping():
    hf = _hf_model()
    cfg = config_from_hf(hf.config)
    assert (cfg.hidden, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab_size) == \
        (256, 2, 4, 2, 128, 512, 512)
    assert cfg.rope_theta == 500000.0 and cfg.rms_eps == 1e-5


def test_loaded_model_matches_transformers_forward():
    hf = _hf_model()
    model = from_hf(hf, device=CPU)
    ids = torch.randint(0, 512, (2, 40), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        out = hf(input_ids=ids, output_hidden_states=True)
        ref_hidden = out.hidden_states[-1].reshape(-1, 256)          # after the final norm
        ref_logp = torch.log_softmax(out.logits.float(), -1).gather(-1, ids[..., None])[..., 0]
        mine_hidden = model.hidden_states(ids)[: ids.numel()].float()
        mine_logp = model.token_logp(ids, ids)
    assert (mine_hidden - ref_hidden).abs().max().item() < 0.04 * ref_hidden.abs().max().item()
    assert (mine_logp - ref_logp).abs().max().item() < 0.05
    # and back: the exported state dict is the one that was loaded
    back = to_hf_state_dict(model)
    ref_state = hf.state_dict()
    assert set(back) == {k for k in ref_state if "rotary" not in k}
    assert all(torch.equal(back[k].float(), ref_state[k].float()) for k in back)


def _tp_worker(rank, world, port, out_dir):
    import os
    import sys

    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from kernel_align_b200.parallel.tp_gemm import TPContext

    model = from_hf(_hf_model(), tp=TPContext(device=CPU), device=CPU)
    ids = torch.randint(0, 512, (2, 40), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        logp = model.token_logp(ids, ids)
    full = to_hf_state_dict(model)                 # every rank reassembles the whole checkpoint
    ref_state = _hf_model().state_dict()
    assert all(torch.equal(full[k].float(), ref_state[k].float()) for k in full)
    torch.save(logp, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_loading_matches_transformers_forward(tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_tp_worker, args=(2, 29811, str(tmp_path)), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "r0.pt"), torch.load(tmp_path / "r1.pt")
    assert torch.equal(a, b)
    hf = _hf_model()
    ids = torch.randint(0, 512, (2, 40), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = torch.log_softmax(hf(input_ids=ids).logits.float(), -1).gather(-1, ids[..., None])[..., 0]
    assert (a - ref).abs().max().item() < 0.05


def test_save_and_load_pretrained_directory(tmp_path):
    from kernel_align_b200.models.hf_convert import load_pretrained, save_pretrained

    hf = _hf_model()
    model = from_hf(hf, device=CPU)
    save_pretrained(model, str(tmp_path / "ckpt"))
    again = load_pretrained(str(tmp_path / "ckpt"), device=CPU)
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), again.named_parameters()):
        assert n1 == n2 and torch.equal(p1, p2), n1
    reloaded = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ckpt"))
    ids = torch.randint(0, 512, (1, 16), generator=torch.Generator().manual_seed(4))
    with torch.no_grad():
        a = hf(input_ids=ids).logits.float()
        b = reloaded(input_ids=ids).logits.float()
    assert (a - b).abs().max().item() < 0.05
