"""TEST INFRASTRUCTURE: seeded inputs for the caller-side kernels (start-of-decoding state, gather tree,
finalize, archive of unfinished beams) and drivers that run them through the product library, the CPU
restatement and the compiled reference.  All drivers take and return numpy arrays."""
import ctypes as C

import numpy as np

SENTINEL = -7


# ------------------------------------------------------------------------------------------------ cases
def gather_tree_case(seed, B, K, T, M=0, prefix=False, virtual=False, final_step=0, bad_parents=False,
                     with_output=True, with_response=False, vocab=12):
    """Inputs of one gatherTree call.  M = 0 stands for the short overloads (no input lengths)."""
    rng = np.random.default_rng(seed)
    c = {"B": B, "K": K, "T": T, "final_step": final_step}
    c["step_ids"] = rng.integers(0, vocab, size=(T, B, K)).astype(np.int32)
    par = rng.integers(0, K, size=(T, B, K)).astype(np.int32)
    if bad_parents:
        par[rng.random(size=par.shape) < 0.02] = -3
    c["parent_ids"] = par if K > 1 or seed % 2 else None
    c["end_tokens"] = rng.integers(0, vocab, size=B).astype(np.int32)
    P = 0
    c["prefix"] = c["virtual"] = c["input_lengths"] = None
    if M > 0:
        if prefix:
            c["prefix"] = rng.integers(0, 4, size=B).astype(np.int32)
            P = 3
        vmax = 0
        if virtual:
            c["virtual"] = rng.integers(0, 3, size=B).astype(np.int32)
            vmax = 2
        lo = (c["prefix"] if prefix else np.zeros(B, np.int32)) + (c["virtual"] if virtual else 0) + 1
        per_entry = np.array([rng.integers(lo[b], M + 1) for b in range(B)], np.int32)
        c["input_lengths"] = np.repeat(per_entry, K).reshape(B, K).astype(np.int32)   # tiled per beam
        c["max_input_length"] = M
        c["max_input_without_prompt_length"] = M - vmax
    else:
        c["max_input_length"] = 1
        c["max_input_without_prompt_length"] = 0 if not with_output else 1
    c["max_prefix"] = P
    low = max(M, 1)
    c["seq_lengths"] = rng.integers(low, T - final_step + 1, size=(B, K)).astype(np.int32)
    c["with_output"] = with_output
    c["with_response"] = with_response
    return c


def finalize_case(seed, B, K, L, with_log_probs=True, short_archives=False):
    rng = np.random.default_rng(seed)
    c = {"B": B, "K": K, "L": L}
    c["topk_output_ids"] = rng.integers(0, 1000, size=(B, 2 * K, L + 1)).astype(np.int32)
    c["topk_sequence_lengths"] = rng.integers(0, L + 1, size=(B, 2 * K)).astype(np.int32)
    c["scores"] = (rng.integers(-40, 0, size=(B, 2 * K)) / 8.0).astype(np.float32)       # ties on purpose
    c["topk_cum_log_probs"] = rng.normal(size=(B, 2 * K)).astype(np.float32)
    c["topk_log_probs"] = rng.normal(size=(B, 2 * K, L + 1)).astype(np.float32) if with_log_probs else None
    lo = 1 if short_archives else K
    c["num_beams"] = rng.integers(lo, 2 * K + 1, size=B).astype(np.int32)
    return c


def insert_case(seed, B, K, L, with_log_probs=True, length_penalty=0.0):
    rng = np.random.default_rng(seed)
    c = {"B": B, "K": K, "L": L, "length_penalty": length_penalty}
    c["output_ids_src"] = rng.integers(0, 1000, size=(L + 1, B * K)).astype(np.int32)
    c["parent_ids_src"] = rng.integers(0, K, size=(L + 1, B * K)).astype(np.int32)
    c["sequence_lengths_src"] = rng.integers(1, L + 1, size=B * K).astype(np.int32)
    c["log_probs_src"] = rng.normal(size=(L + 1, B * K)).astype(np.float32) if with_log_probs else None
    c["finished"] = (rng.random(size=B * K) < 0.3).astype(np.uint8)
    c["cum_log_probs"] = (-rng.random(size=B * K) * 20).astype(np.float32)
    c["num_beams"] = rng.integers(0, K, size=B).astype(np.int32)
    c["is_done"] = (rng.random(size=B) < 0.25).astype(np.uint8)
    return c


# ------------------------------------------------------------------------------------------------ drivers
class _Host:
    """numpy arrays passed by pointer"""
    name = "host"

    def put(self, a):
        return None if a is None else np.ascontiguousarray(a).copy()

    def ptr(self, a):
        return None if a is None else a.ctypes.data

    def get(self, a):
        return a

    def sync(self):
        pass


class _Device:
    """torch CUDA tensors passed by pointer"""
    name = "device"

    def put(self, a):
        import torch
        return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()

    def ptr(self, a):
        return None if a is None else a.data_ptr()

    def get(self, a):
        return a.cpu().numpy()

    def sync(self):
        import torch
        torch.cuda.synchronize()


def run_gather_tree(impl, c):
    """impl: 'oracle' | 'ours' | 'ref'.  Returns dict(beams, lengths, output_ids, response)."""
    from fastertransformer_b200._abi import GatherTreeParams
    m = _Host() if impl == "oracle" else _Device()
    B, K, T = c["B"], c["K"], c["T"]
    trimmed = c["max_prefix"] + (c["max_input_length"] - c["max_input_without_prompt_length"])
    out_len = T - trimmed
    beams = m.put(np.full((T, B, K), SENTINEL, np.int32))
    lengths = m.put(c["seq_lengths"])
    out = m.put(np.full((B, K, max(out_len, 1)), SENTINEL, np.int32)) if c["with_output"] else None
    resp = m.put(np.full((B, K), SENTINEL, np.int32)) if c["with_response"] else None
    keep = [m.put(c[k]) for k in ("input_lengths", "step_ids", "parent_ids", "end_tokens", "prefix", "virtual")]
    il, ids, par, end, pre, vir = keep
    if impl == "ref":
        import ft_reference
        rc = ft_reference.ref_lib().ftref_gather_tree(
            m.ptr(beams), m.ptr(lengths), c["final_step"], m.ptr(il), m.ptr(resp), T, B, K, m.ptr(ids), m.ptr(par),
            m.ptr(end), c["max_input_length"], m.ptr(pre), m.ptr(vir), c["max_input_without_prompt_length"],
            c["max_prefix"], m.ptr(out), None)
    else:
        P = GatherTreeParams(
            beams=m.ptr(beams), max_sequence_lengths=m.ptr(lengths), max_sequence_length_final_step=c["final_step"],
            input_lengths=m.ptr(il), response_input_lengths=m.ptr(resp), max_time=T, batch_size=B, beam_width=K,
            step_ids=m.ptr(ids), parent_ids=m.ptr(par), end_tokens=m.ptr(end),
            max_input_length=c["max_input_length"], prefix_soft_prompt_lengths=m.ptr(pre),
            p_prompt_tuning_prompt_lengths=m.ptr(vir),
            max_input_without_prompt_length=c["max_input_without_prompt_length"],
            max_prefix_soft_prompt_length=c["max_prefix"], output_ids=m.ptr(out), stream=None)
        if impl == "oracle":
            from ft_oracle import oracle_lib
            rc = oracle_lib().oracle_gather_tree(C.byref(P))
        else:
            from fastertransformer_b200 import lib
            rc = lib.ftb200_gather_tree(C.byref(P))
    m.sync()
    assert rc == 0, rc
    return {"beams": m.get(beams), "lengths": m.get(lengths),
            "output_ids": None if out is None else m.get(out)[:, :, :out_len],
            "response": None if resp is None else m.get(resp)}


def run_finalize(impl, c):
    m = _Host() if impl == "oracle" else _Device()
    B, K, L = c["B"], c["K"], c["L"]
    out = m.put(np.full((B, K, L), SENTINEL, np.int32))
    lens = m.put(np.full((B, K), SENTINEL, np.int32))
    cum = m.put(np.full((B, K), np.float32(SENTINEL)))
    lp = m.put(np.full((B, K, L), np.float32(SENTINEL))) if c["topk_log_probs"] is not None else None
    ins = [m.put(c[k]) for k in ("topk_output_ids", "topk_sequence_lengths", "scores", "topk_cum_log_probs",
                                 "topk_log_probs", "num_beams")]
    args = [m.ptr(out), m.ptr(lens), m.ptr(cum), m.ptr(lp)] + [m.ptr(a) for a in ins] + [K, L, B]
    if impl == "oracle":
        from ft_oracle import oracle_lib
        rc = oracle_lib().oracle_finalize(*args)
    elif impl == "ref":
        import ft_reference
        rc = ft_reference.ref_lib().ftref_finalize(*args, None)
    else:
        from fastertransformer_b200 import lib
        rc = lib.ftb200_finalize(*args, None)
    m.sync()
    assert rc == 0, rc
    return {"output_ids": m.get(out), "lengths": m.get(lens), "cum": m.get(cum),
            "log_probs": None if lp is None else m.get(lp)}


def run_insert(impl, c):
    from fastertransformer_b200._abi import BeamHyps
    m = _Host() if impl == "oracle" else _Device()
    B, K, L = c["B"], c["K"], c["L"]
    with_lp = c["log_probs_src"] is not None
    ids_t = m.put(np.full((B, 2 * K, L + 1), SENTINEL, np.int32))
    len_t = m.put(np.full((B, 2 * K), SENTINEL, np.int32))
    cum_t = m.put(np.full((B, 2 * K), np.float32(SENTINEL)))
    nrm_t = m.put(np.full((B, 2 * K), np.float32(SENTINEL)))
    lp_t = m.put(np.full((B, 2 * K, L + 1), np.float32(SENTINEL))) if with_lp else None
    nb = m.put(c["num_beams"])
    done = m.put(c["is_done"])
    ins = [m.put(c[k]) for k in ("output_ids_src", "parent_ids_src", "sequence_lengths_src", "log_probs_src")]
    fin, cum = m.put(c["finished"]), m.put(c["cum_log_probs"])
    if impl == "ref":
        import ft_reference
        rc = ft_reference.ref_lib().ftref_insert_unfinished_path(
            m.ptr(ids_t), m.ptr(len_t), m.ptr(cum_t), m.ptr(nrm_t), m.ptr(lp_t), m.ptr(nb), m.ptr(done),
            *[m.ptr(a) for a in ins], L, c["length_penalty"], m.ptr(fin), m.ptr(cum), B, K, None)
    else:
        H = BeamHyps(output_ids_tgt=m.ptr(ids_t), sequence_lengths_tgt=m.ptr(len_t), cum_log_probs=m.ptr(cum_t),
                     normed_scores=m.ptr(nrm_t), log_probs=m.ptr(lp_t), min_normed_scores=None,
                     num_beams=m.ptr(nb), is_done=m.ptr(done), early_stopping=1)
        args = [C.byref(H)] + [m.ptr(a) for a in ins] + [L, c["length_penalty"], m.ptr(fin), m.ptr(cum), B, K]
        if impl == "oracle":
            from ft_oracle import oracle_lib
            rc = oracle_lib().oracle_insert_unfinished_path(*args)
        else:
            from fastertransformer_b200 import lib
            rc = lib.ftb200_insert_unfinished_path(*args, None)
    m.sync()
    assert rc == 0, rc
    return {"output_ids_tgt": m.get(ids_t), "lengths_tgt": m.get(len_t), "cum_tgt": m.get(cum_t),
            "normed": m.get(nrm_t), "log_probs_tgt": None if lp_t is None else m.get(lp_t),
            "num_beams": m.get(nb)}


def run_initialize(impl, B, K, max_input_length, dtype, with_word_ids=True, seed=0):
    """dtype: 0 float, 1 half, 2 bf16.  cum_log_probs comes back as float32."""
    rng = np.random.default_rng(seed)
    sentence_ids = rng.integers(0, 1000, size=B).astype(np.int32)
    m = _Host() if impl == "oracle" else _Device()
    fin = m.put(np.full(B * K, 9, np.uint8))
    seq = m.put(np.full(B * K, SENTINEL, np.int32))
    word = m.put(np.full(B * K, SENTINEL, np.int32)) if with_word_ids else None
    sid = m.put(sentence_ids)
    if impl == "oracle":
        from ft_oracle import oracle_lib
        cum = np.zeros(B * K, np.float32)
        rc = oracle_lib().oracle_decoding_initialize(m.ptr(fin), m.ptr(seq), m.ptr(word), cum.ctypes.data, dtype,
                                                     m.ptr(sid), B, K, max_input_length)
        cum_f = cum
    else:
        import torch
        tdt = [torch.float32, torch.float16, torch.bfloat16][dtype]
        cum = torch.full((B * K,), 3.0, dtype=tdt, device="cuda")
        if impl == "ref":
            import ft_reference
            f = ft_reference.ref_lib().ftref_decoding_initialize
        else:
            from fastertransformer_b200 import lib
            f = lib.ftb200_decoding_initialize
        rc = f(m.ptr(fin), m.ptr(seq), m.ptr(word), cum.data_ptr(), dtype, m.ptr(sid), B, K, max_input_length, None)
        m.sync()
        cum_f = cum.float().cpu().numpy()
    assert rc == 0, rc
    return {"finished": m.get(fin), "sequence_length": m.get(seq),
            "word_ids": None if word is None else m.get(word), "cum": cum_f}


def same(a, b, float_keys=()):
    """Asserts two result dicts are equal: integers bit for bit, floats listed in float_keys to 1e-6 relative."""
    assert a.keys() == b.keys()
    for k in a:
        if a[k] is None or b[k] is None:
            assert a[k] is None and b[k] is None, k
        elif k in float_keys:
            np.testing.assert_allclose(a[k], b[k], rtol=2e-6, atol=0, err_msg=k)
        else:
            np.testing.assert_array_equal(a[k], b[k], err_msg=k)


# Small cases whose reference outputs are committed under tests/golden/decoding_ref.json.
GOLDEN_GATHER = {
    "short_overload": dict(seed=1, B=3, K=4, T=9, with_output=False),
    "gpt_beams": dict(seed=2, B=4, K=4, T=14, M=5, final_step=1, with_response=True),
    "gpt_sampling": dict(seed=4, B=6, K=1, T=12, M=4, final_step=1),
    "prefix_prompt": dict(seed=5, B=4, K=2, T=16, M=6, prefix=True, final_step=1, with_response=True),
    "virtual_prompt": dict(seed=7, B=2, K=8, T=13, M=5, virtual=True, final_step=1),
    "bad_parents": dict(seed=9, B=5, K=4, T=20, M=3, final_step=1, bad_parents=True),
}
GOLDEN_FINALIZE = {
    "k4": dict(seed=11, B=3, K=4, L=9),
    "k1_no_log_probs": dict(seed=12, B=5, K=1, L=6, with_log_probs=False),
    "k20": dict(seed=13, B=2, K=20, L=5),
}
GOLDEN_INSERT = {
    "k4": dict(seed=21, B=4, K=4, L=10),
    "k2_length_penalty": dict(seed=22, B=6, K=2, L=7, length_penalty=0.8, with_log_probs=False),
    "k16": dict(seed=23, B=3, K=16, L=12, length_penalty=1.5),
}
