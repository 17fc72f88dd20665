"""The benchmarked composition at its own shape: Llama-3-8B (32 layers, hidden 4096, 32 query / 8 KV heads, FFN
14336, vocabulary 128256), bf16 weights N(0, 0.02), fused weight-streaming kernels, TMA decode attention, decode
steps replayed from a CUDA graph -- against the fp32 oracle holding the SAME weight values.

The context is shortened to 8192 tokens (the decode step's kernels and their composition are the same at any
length).  The oracle's fp32 torch code runs on the GPU here -- a CPU run of an 8B model is out of reach -- and stays
what it is: the checker.  The package's caches take over the oracle's prefilled K/V (rounded to bf16), so that the
comparison is about the decode path, from identical prompts.

What is checked, per decode step (the oracle's greedy token is fed to both sides):

1. LAYER BY LAYER, every layer given the oracle's own input: the residual stream that enters layer i in the oracle
   (rounded to bf16) goes through the package's layer i -- fused norm + QKV + RoPE + append, decode attention
   (+ selection scores and top-k on the filter layers), output projection, gate/up + SiLU, down projection -- and
   must leave it within 2e-2 x max(1, largest magnitude of the oracle's output) of the oracle's output; the final
   norm + lm_head + arg-max kernel, given the oracle's last hidden state, must give its logits within 2e-2.
2. SELECTION: each filter layer's index list is exactly the top-k of the package's own fp32 score tensor, and
   differs from the oracle's list only on positions whose oracle score lies within (twice the largest score
   difference between the two pipelines + 1e-4) of the oracle's k-th score.
3. COMPOSITION: the free-running step replayed from a CUDA graph gives bit for bit the logits of the same step
   launched eagerly.
4. REPORTED, not bounded by 2e-2: the free-running logits and the per-layer growth of the difference.  A 16-bit
   residual stream rounds every layer's output to 8 mantissa bits; through 32 random-weight layers those
   roundings compound (two correct 16-bit pipelines that round at different points drift apart just as much), so
   the free-running difference from an fp32 run is of the order of 0.5 in logits of magnitude about 5.  The test
   prints it with its growth per layer and only requires the growth to be gradual (no layer adds more than 0.1 of
   the stream's magnitude).
"""
from types import SimpleNamespace

import pytest
import torch

from oracle.llama_oracle import OracleLM
from parity import band_check

pytestmark = pytest.mark.gpu

CTX, STEPS = 8192, 12


@torch.no_grad()
def test_llama3_8b_shape_fused_graph_decode_matches_fp32_oracle():
    import oracle as orc
    from omnikv_b200 import ops
    from omnikv_b200.modeling import LlamaCompressorConfig, OmniKVMulLM
    from omnikv_b200.modeling.omnikv import DecodeRunner
    if torch.cuda.get_device_properties(0).total_memory < 100 * 2 ** 30:
        pytest.skip("needs about 70 GB of device memory (bf16 model + its fp32 oracle)")
    bf = torch.bfloat16
    cfg = LlamaCompressorConfig()  # the Llama-3-8B shape
    cfg.set_config_of_compressor(model_cls="multi", cache_cls="multi", do_select_layers="2,8,18", num_wait_load_layers=1,
                                 real_offload=False, dense_more=True, num_of_selected_tokens=0.067, selector_cls="last",
                                 window_size=16, fused_decode=True)
    lm = OmniKVMulLM.from_config(cfg, dtype=bf, device="cuda", seed=0)
    ref = OracleLM(cfg.to_dict(), lm.hf_state_dict(), device="cuda")
    n_layers, filters = cfg.num_hidden_layers, (2, 8, 18)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (1, CTX), generator=g)
    lo, oc = ref.forward(ids)

    def take_over():  # a package cache holding the oracle's prompt K/V
        filled = SimpleNamespace(key_cache=[k.to(bf) for k in oc.key_cache], value_cache=[v.to(bf) for v in oc.value_cache],
                                 _seen_tokens=CTX)
        c = lm.new_cache(filled)
        c.stage = "decoding"
        return c

    cache_graph, cache_eager, cache_forced = take_over(), take_over(), take_over()
    tok = lo[:, -1].argmax(-1, keepdim=True)
    runner = None
    hbuf = torch.zeros(cfg.hidden_size, dtype=bf, device="cuda")
    logits_k = torch.empty(1, cfg.vocab_size, dtype=torch.float32, device="cuda")
    best = torch.zeros(1, dtype=torch.int64, device="cuda")
    token_k = torch.zeros(1, 1, dtype=torch.int64, device="cuda")
    dummy_pos = object()  # the fused path rotates inside its QKV kernel and never looks at the table
    free_err, layer_err, logit_err, growth, sel_report = [], [], [], None, []
    for s in range(STEPS):
        lo, oc = ref.forward(tok, oc, fwd_no=s)
        want, trace = lo[:, -1], ref.hidden_trace

        # --- free-running, replayed from a CUDA graph (the first step runs eagerly and sets everything up) ---
        if runner is None:
            runner = DecodeRunner(lm, None, cache=cache_graph, first_token=tok, max_new_tokens=STEPS + 2,
                                  use_cuda_graph=True, warmup_steps=1)
            assert runner.graph is not None
            assert lm.model.layers[0]._fused_ok(torch.zeros(1, 1, cfg.hidden_size, dtype=bf, device="cuda"))
        else:
            runner.token.copy_(tok)
            runner.run(1)
        graph_logits = runner.logits.clone()
        free_err.append((graph_logits.view(-1) - want.view(-1)).abs().max().item())

        # --- the same step launched eagerly, with every layer's output recorded ---
        rec = []
        hooks = [layer.register_forward_hook(lambda m, i, o: rec.append(o[0].float().clone())) for layer in lm.model.layers]
        eager_logits, _ = lm._decode_step(tok, cache_eager)
        for h in hooks:
            h.remove()
        assert torch.equal(eager_logits.view(-1), graph_logits.view(-1)), s
        rel = [((rec[i].view(-1) - trace[i + 1].view(-1)).abs().max() / trace[i + 1].abs().max()).item() for i in range(n_layers)]
        growth = rel if growth is None else [max(a, b) for a, b in zip(growth, rel)]

        # --- layer by layer, every layer fed the oracle's input ---
        cache_forced.begin_decode_step()
        for i, layer in enumerate(lm.model.layers):
            hbuf.copy_(trace[i].view(-1))
            out = layer(hbuf.view(1, 1, -1), past_key_value=cache_forced, position_embeddings=dummy_pos)[0]
            err = (out.float().view(-1) - trace[i + 1].view(-1)).abs().max().item()
            mag = trace[i + 1].abs().max().item()
            layer_err.append(err / max(1.0, mag))
            assert err <= 2e-2 * max(1.0, mag), (s, i, err, mag)
        hbuf.copy_(trace[n_layers].view(-1))
        ops.decode_logits(hbuf, lm.model.norm.weight, lm.model.norm.variance_epsilon, lm.lm_head.weight, 0, logits_k, best, token_k)
        logit_err.append((logits_k.view(-1) - want.view(-1)).abs().max().item())
        assert logit_err[-1] <= 2e-2, (s, logit_err[-1])
        for f in filters:
            st = cache_forced.sel_state[f]
            planes = st.planes.max(dim=0).values[0]            # the package's own fp32 scores [P]
            mine = st.idx[0, : st.count.item()].cpu()
            k = int(st.k0.item())
            assert torch.equal(mine.long(), orc.topk_ascending(planes[None].cpu(), k)[0]), (s, f)
            scores, k_sel = ref.scores[(s, f)]
            assert k_sel == k
            score_err = (planes[:CTX] - scores[0]).abs().max().item()
            n_diff = band_check(scores[0], k, mine.tolist(), ref.selected[(s, f)][0].tolist(), 2 * score_err + 1e-4, (s, f))
            sel_report.append((s, f, round(score_err, 5), n_diff))
        tok = want.argmax(-1, keepdim=True)
    ops.check_status("cuda")
    print("layer by layer (oracle's input): largest |out - oracle| / max(1, |oracle|):", round(max(layer_err), 5),
          "; logits from the oracle's last hidden state:", round(max(logit_err), 5))
    print("selection (step, filter layer, largest score difference, positions that differ of %d):" % k, sel_report[-6:])
    print("free-running |logit - oracle| per step:", [round(e, 3) for e in free_err])
    print("free-running growth per layer (largest |stream - oracle| / largest |oracle|):", [round(r, 4) for r in growth])
    steps_up = [growth[0]] + [growth[i] - growth[i - 1] for i in range(1, n_layers)]
    assert max(steps_up) <= 0.1, steps_up
