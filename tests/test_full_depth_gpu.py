"""The benchmarked composition at its own shape: Llama-3-8B (32 layers, hidden 4096, 32 query / 8 KV heads, FFN
14336, vocabulary 128256), bf16 weights N(0, 0.02), fused weight-streaming kernels, TMA decode attention, decode
steps replayed from a CUDA graph -- against the fp32 oracle holding the SAME weight values.

The context is shortened to 8192 tokens (a real prefill; the decode step's kernels and their composition are the
same at any length).  The oracle's fp32 torch code runs on the GPU here -- a CPU run of an 8B model is out of reach
-- and stays what it is: the checker.

Tolerances.  Logits: 2e-2 absolute against the fp32 oracle, teacher-forced (the oracle's greedy token is fed to
both).  Selection: the package's index list must be exactly the top-k of ITS OWN fp32 score tensor (bit-exact
top-k on identical scores), and may differ from the oracle's list only on positions whose oracle score lies within
(twice the largest score difference between the two pipelines + 1e-4) of the oracle's k-th score: a 16-bit pipeline
rounds q and K, so its scores differ from fp32 ones by about 1e-2 and positions that close to the threshold are
interchangeable.
"""
import pytest
import torch

from oracle.llama_oracle import OracleLM
from parity import band_check

pytestmark = pytest.mark.gpu

CTX, STEPS = 8192, 16


def test_llama3_8b_shape_fused_graph_decode_matches_fp32_oracle():
    import oracle as orc
    from omnikv_b200 import ops
    from omnikv_b200.modeling import LlamaCompressorConfig, OmniKVMulLM
    from omnikv_b200.modeling.omnikv import DecodeRunner
    if torch.cuda.get_device_properties(0).total_memory < 100 * 2 ** 30:
        pytest.skip("needs about 70 GB of device memory (bf16 model + its fp32 oracle)")
    cfg = LlamaCompressorConfig()  # the Llama-3-8B shape
    cfg.set_config_of_compressor(model_cls="multi", cache_cls="multi", do_select_layers="2,8,18", num_wait_load_layers=1,
                                 real_offload=False, dense_more=True, num_of_selected_tokens=0.067, selector_cls="last",
                                 window_size=16, fused_decode=True)
    lm = OmniKVMulLM.from_config(cfg, dtype=torch.bfloat16, device="cuda", seed=0)
    ref = OracleLM(cfg.to_dict(), lm.hf_state_dict(), device="cuda")
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (1, CTX), generator=g)

    # the oracle: prefill, then STEPS greedy decode forwards
    lo, oc = ref.forward(ids)
    want, toks = [lo[:, -1]], []
    for s in range(STEPS):
        toks.append(want[-1].argmax(-1, keepdim=True))
        lo, oc = ref.forward(toks[-1], oc, fwd_no=s)
        want.append(lo[:, -1])
    torch.cuda.synchronize()

    # the package: prefill, one eager decode step (first-use set-up), the rest replayed from a CUDA graph
    out = lm(input_ids=ids.cuda())
    cache = out.past_key_values
    cache.reserve = max(cache.reserve, STEPS + 8)
    errs = [(out.logits[:, -1] - want[0]).abs().max().item()]
    runner = DecodeRunner(lm, None, cache=cache, first_token=toks[0], max_new_tokens=STEPS + 2, use_cuda_graph=True,
                          warmup_steps=1)
    assert runner.graph is not None and lm.model.layers[0]._fused_ok(torch.zeros(1, 1, 4096, dtype=torch.bfloat16, device="cuda"))
    sel_report = []
    for s in range(STEPS):
        if s > 0:
            runner.token.copy_(toks[s])
            runner.run(1)
        torch.cuda.synchronize()
        errs.append((runner.logits - want[s + 1]).abs().max().item())
        for f in (2, 8, 18):
            st = cache.sel_state[f]
            planes = st.planes.max(dim=0).values[0]            # the package's own fp32 scores [P]
            mine = st.idx[0, : st.count.item()].cpu()
            k = int(st.k0.item())
            # (1) bit-exact top-k of the package's own score tensor
            assert torch.equal(mine.long(), orc.topk_ascending(planes[None].cpu(), k)[0]), (s, f)
            # (2) against the oracle's selection, up to the score difference of the two pipelines
            scores, k_sel = ref.scores[(s, f)]
            assert k_sel == k
            score_err = (planes[:CTX] - scores[0]).abs().max().item()
            n_diff = band_check(scores[0], k, mine.tolist(), ref.selected[(s, f)][0].tolist(), 2 * score_err + 1e-4, (s, f))
            sel_report.append((s, f, round(score_err, 5), n_diff))
    ops.check_status("cuda")
    print("max |logit - oracle| per forward (prefill, then decode steps):", [round(e, 5) for e in errs])
    print("selection (step, filter layer, max score difference, positions that differ of %d):" % k, sel_report[-6:])
    assert max(errs[1:]) <= 2e-2, errs
