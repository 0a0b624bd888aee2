"""Unit tests of speculative decoding's host parts - the accept/reject rule, the n-gram and self-draft proposers - and
of the host sampler (the shape of the reference's tests/test_speculative.py: greedy and stochastic verification,
n-gram, self-draft, truncation, a simulated cycle).  Target distributions are made up on the spot; no model runs."""
import collections
import random

import numpy as np
import pytest
import torch

from zse_b200.sched.draft_model import DraftModel, NGramDraftModel, SelfDraftModel, make_draft_model
from zse_b200.sched.sampler import Sampler
from zse_b200.sched.verifier import (SpeculativeVerifier, VerifyResult, acceptance_rate, effective_tokens_per_step)


def onehot(v, i):
    t = torch.zeros(v)
    t[i] = 1.0
    return t


# ---- greedy verification ----------------------------------------------------------------------------------------
def test_greedy_accepts_the_matching_prefix_and_adds_the_targets_next_token():
    v = SpeculativeVerifier()
    r = v.verify_greedy([5, 6, 7], [5, 6, 7, 8])
    assert (r.accepted_tokens, r.num_drafted, r.num_accepted) == ([5, 6, 7, 8], 3, 3)       # all + bonus
    r = v.verify_greedy([5, 6, 7], [5, 9, 7, 8])
    assert (r.accepted_tokens, r.num_accepted) == ([5, 9], 1)                               # corrected at the mismatch
    r = v.verify_greedy([5, 6, 7], [1, 6, 7, 8])
    assert (r.accepted_tokens, r.num_accepted) == ([1], 0)
    r = v.verify_greedy([], [4])
    assert (r.accepted_tokens, r.num_drafted, r.num_accepted, r.acceptance_rate) == ([4], 0, 0, 0.0)


def test_a_later_match_after_a_mismatch_does_not_count():
    r = SpeculativeVerifier().verify_greedy([1, 2, 3], [1, 0, 3, 9])
    assert r.accepted_tokens == [1, 0] and r.num_accepted == 1


def test_verifier_statistics_accumulate():
    v = SpeculativeVerifier()
    v.verify_greedy([1, 2], [1, 2, 3])
    v.verify_greedy([1, 2], [0, 2, 3])
    assert v.stats() == {"steps": 2, "drafted": 4, "accepted": 2, "acceptance_rate": 0.5}
    assert SpeculativeVerifier().stats()["acceptance_rate"] == 0.0
    assert VerifyResult([1], 4, 3).acceptance_rate == 0.75
    assert acceptance_rate(2, 4) == 0.5 and acceptance_rate(1, 0) == 0.0
    assert effective_tokens_per_step(3) == 3.0


# ---- stochastic verification ------------------------------------------------------------------------------------
def test_identical_distributions_accept_every_draft():
    V = 8
    p = torch.softmax(torch.randn(V, generator=torch.Generator().manual_seed(0)), 0)
    v = SpeculativeVerifier(seed=1)
    for _ in range(20):
        r = v.verify_stochastic([3, 4], [p, p], [p, p, p])
        assert r.num_accepted == 2 and r.accepted_tokens[:2] == [3, 4] and len(r.accepted_tokens) == 3


def test_a_draft_the_target_gives_no_mass_is_always_replaced_from_the_residual():
    V = 6
    q = onehot(V, 2)                       # the draft is sure of token 2
    p = torch.tensor([0.0, 0.5, 0.0, 0.5, 0.0, 0.0])
    v = SpeculativeVerifier(seed=3)
    seen = collections.Counter()
    for _ in range(200):
        r = v.verify_stochastic([2], [q], [p, p])
        assert r.num_accepted == 0 and len(r.accepted_tokens) == 1
        seen[r.accepted_tokens[0]] += 1
    assert set(seen) == {1, 3} and min(seen.values()) > 60                                   # max(0, p - q) = p here


def test_a_draft_with_zero_proposal_probability_is_taken_if_the_target_allows_it():
    V = 4
    q = onehot(V, 0)                       # q(1) = 0
    p = onehot(V, 1)
    r = SpeculativeVerifier(seed=0).verify_stochastic([1], [q], [p, onehot(V, 3)])
    assert r.accepted_tokens == [1, 3] and r.num_accepted == 1
    # neither gives it mass: replaced from the target
    r = SpeculativeVerifier(seed=0).verify_stochastic([2], [q], [p, p])
    assert r.accepted_tokens == [1] and r.num_accepted == 0


def test_rejection_sampling_reproduces_the_target_distribution():
    """The point of the rule: whatever the draft proposes, the first emitted token follows the target."""
    V = 5
    p = torch.tensor([0.05, 0.4, 0.3, 0.05, 0.2])
    q = torch.tensor([0.5, 0.1, 0.1, 0.2, 0.1])
    rng = random.Random(7)
    v = SpeculativeVerifier(seed=11)
    counts = np.zeros(V)
    n = 6000
    for _ in range(n):
        d = rng.choices(range(V), weights=q.tolist())[0]
        r = v.verify_stochastic([d], [q], [p, p])
        counts[r.accepted_tokens[0]] += 1
    assert np.abs(counts / n - p.numpy()).max() < 0.025
    assert 0.3 < v.stats()["acceptance_rate"] < 0.9


def test_stochastic_stops_at_the_first_rejection():
    V = 4
    p_ok, p_no = onehot(V, 1), onehot(V, 3)
    q = onehot(V, 1)
    r = SpeculativeVerifier(seed=0).verify_stochastic([1, 1, 1], [q, q, q], [p_ok, p_no, p_ok, p_ok])
    assert r.accepted_tokens == [1, 3] and r.num_accepted == 1 and r.num_drafted == 3


# ---- the reference's entry point --------------------------------------------------------------------------------
def test_verify_and_accept_takes_fp16_bytes_and_tensors():
    V = 10
    rows = []
    for best in (4, 7, 2):
        x = np.full(V + 6, -5.0, dtype=np.float16)       # padded rows: only the first `vocab_size` entries count
        x[best] = 5.0
        x[V + 1] = 50.0
        rows.append(x.tobytes())
    v = SpeculativeVerifier()
    toks, n = v.verify_and_accept([4, 7], None, rows, V, temperature=0.0)
    assert (toks, n) == ([4, 7, 2], 2)
    toks, n = v.verify_and_accept([4, 1], None, [torch.from_numpy(np.frombuffer(r, dtype=np.float16).copy()) for r in rows],
                                  V, temperature=0.0)
    assert (toks, n) == ([4, 7], 1)
    with pytest.raises(ValueError):
        v.verify_and_accept([4, 7], None, rows[:2], V, temperature=0.0)


def test_verify_and_accept_with_temperature_uses_the_softmax_of_the_rows():
    V = 6
    sharp = torch.full((V,), -30.0)
    sharp[2] = 30.0
    draft = onehot(V, 2).tolist()
    toks, n = SpeculativeVerifier(seed=5).verify_and_accept([2, 2], [draft, draft], [sharp, sharp, sharp], V, 0.7)
    assert (toks, n) == ([2, 2, 2], 2)


# ---- n-gram proposer --------------------------------------------------------------------------------------------
def test_ngram_proposes_what_followed_the_latest_occurrence_of_the_suffix():
    m = NGramDraftModel(n=3)
    m.reset([1, 2, 3, 4, 9, 1, 2, 5, 6, 7, 1, 2])
    assert m.propose(3) == [5, 6, 7]                      # the later "1 2", not the first one
    assert m.propose(1) == [5] and len(m) == 12
    m.extend([5])
    assert m.propose(4) == [6, 7, 1, 2]                   # suffix "2 5" -> continues through the context


def test_ngram_falls_back_to_a_shorter_suffix_and_gives_up_without_a_match():
    m = NGramDraftModel(n=4, min_n=2)
    m.reset([7, 8, 9, 3, 4, 5, 6, 1, 9])                  # no earlier "6 1 9", no "1 9"; "9" was followed by 3
    assert m.propose(2) == [3, 4]
    m.reset([1, 2, 3, 4])
    assert m.propose(3) == []
    m.reset([])
    assert m.propose(3) == [] and len(m) == 0
    with pytest.raises(ValueError):
        NGramDraftModel(n=1)


def test_ngram_incremental_extension_equals_a_rebuild_and_truncate_forgets():
    rng = random.Random(0)
    seq = [rng.randrange(6) for _ in range(200)]
    inc = NGramDraftModel(n=3)
    inc.reset(seq[:50])
    for i in range(50, 200, 7):
        inc.extend(seq[i:i + 7])
        fresh = NGramDraftModel(n=3)
        fresh.reset(seq[:min(i + 7, 200)])
        assert inc.propose(4) == fresh.propose(4)
    inc.truncate(120)                                     # rejected drafts are dropped
    fresh = NGramDraftModel(n=3)
    fresh.reset(seq[:120])
    assert len(inc) == 120 and inc.propose(4) == fresh.propose(4)
    inc.truncate(500)                                     # longer than the context: nothing happens
    assert len(inc) == 120
    inc.update([1, 2])                                    # the reference's name for extend
    assert len(inc) == 122


def test_generate_drafts_always_returns_k_tokens_with_distributions():
    m = NGramDraftModel(vocab_size_val=16, n=3, confidence=0.8)
    drafts, probs = m.generate_drafts([1, 2, 3, 1, 2], 4)
    assert drafts == [3, 1, 2, 2]                         # three found, the last one repeated to fill
    assert len(probs) == 4 and all(len(p) == 16 for p in probs)
    assert abs(sum(probs[0]) - 1.0) < 1e-9 and probs[0][3] == 0.8 and probs[0][0] == pytest.approx(0.2 / 15)
    drafts, probs = m.generate_drafts([4, 5, 6], 2)       # nothing to look up: the last context token is the guess
    assert drafts == [6, 6] and probs[0][6] == 0.8
    assert m.vocab_size() == 16
    drafts, _ = NGramDraftModel().generate_drafts([], 3)
    assert drafts == [0, 0, 0]


def test_self_draft_repeats_the_last_token():
    m = SelfDraftModel(vocab_size_val=8)
    assert m.propose(3) == []
    m.reset([4, 5])
    assert m.propose(3) == [5, 5, 5]
    m.extend([7])
    m.extend([])
    assert m.propose(2) == [7, 7]
    m.truncate(0)                                         # keeps no history to truncate
    assert m.propose(1) == [7]
    logits = np.zeros(8, dtype=np.float16)
    logits[6] = 3.0
    m.set_last_logits(logits.tobytes())
    assert m.propose(2) == [6, 6]
    m.set_last_logits(b"")
    assert m.propose(1) == [6]
    drafts, probs = m.generate_drafts([1, 2], 2)
    assert drafts == [2, 2] and probs[0][2] == 0.9


def test_make_draft_model():
    assert isinstance(make_draft_model("ngram"), NGramDraftModel)
    assert isinstance(make_draft_model("self"), SelfDraftModel)
    assert isinstance(make_draft_model("self"), DraftModel)
    with pytest.raises(ValueError):
        make_draft_model("medusa")


def test_a_simulated_cycle_emits_exactly_the_targets_greedy_sequence():
    """Draft, verify, append, truncate - whatever the proposer guesses, greedy verification yields the target's own
    sequence, in fewer steps when the guesses are good."""
    target = [1, 2, 3, 1, 2, 3, 1, 2, 3, 4, 4, 4, 4, 1, 2, 3, 1, 2, 9]

    def target_argmax(prefix_len, drafts):
        # what the target would emit after prefix + drafts[:i], for i = 0..len(drafts): it follows `target` as long as
        # the drafts did, anything else derails it (returns a token the sequence never contains)
        out = []
        ok = True
        for i in range(len(drafts) + 1):
            pos = prefix_len + i
            out.append(target[pos] if ok and pos < len(target) else 0)
            if i < len(drafts) and (pos >= len(target) or drafts[i] != target[pos]):
                ok = False
        return out

    for mode in ("ngram", "self"):
        m = make_draft_model(mode)
        v = SpeculativeVerifier()
        seq = target[:3]
        m.reset(seq)
        steps = 0
        while len(seq) < len(target):
            drafts = m.propose(4)[: len(target) - len(seq) - 1]
            r = v.verify_greedy(drafts, target_argmax(len(seq), drafts))
            seq += r.accepted_tokens
            m.extend(r.accepted_tokens)
            steps += 1
        assert seq == target
        assert steps <= len(target) - 3
        if mode == "ngram":
            assert steps < len(target) - 3 and v.stats()["accepted"] > 0       # the repeats were worth drafting


# ---- host sampler ----------------------------------------------------------------------------------------------
def test_sampler_greedy_cases():
    x = torch.tensor([0.1, 2.0, -1.0, 1.9])
    s = Sampler(seed=0)
    assert Sampler.greedy(x) == 1 and s.sample(x, temperature=0.0) == 1 and s.sample(x, top_k=1) == 1
    assert s.sample(x.half().numpy(), temperature=0.0) == 1                      # arrays and half precision are fine


def test_sampler_seed_makes_draws_repeatable():
    x = torch.randn(50, generator=torch.Generator().manual_seed(1))
    a = [Sampler(seed=3).sample(x, temperature=1.0) for _ in range(3)]
    assert len(set(a)) == 1
    s = Sampler(seed=3)
    assert s.sample(x, seed=99) == s.sample(x, seed=99)                          # a per-call seed overrides the stream
    draws = {Sampler(seed=i).sample(x, temperature=1.5) for i in range(40)}
    assert len(draws) > 5


def test_top_k_and_top_p_restrict_the_support():
    x = torch.tensor([5.0, 4.0, 3.0, 0.0, -1.0, -2.0])
    s = Sampler(seed=0)
    assert {s.sample(x, temperature=2.0, top_k=2) for _ in range(200)} == {0, 1}
    assert {s.sample(x, temperature=1.0, top_p=0.5) for _ in range(100)} == {0}   # the first token alone reaches 0.5
    wide = {s.sample(x, temperature=3.0) for _ in range(600)}
    assert wide == {0, 1, 2, 3, 4, 5}


def test_repetition_penalty_moves_mass_away_from_seen_tokens():
    x = torch.tensor([2.0, 2.0])
    s = Sampler(seed=0)
    n = 2000
    base = sum(s.sample(x, temperature=1.0) == 0 for _ in range(n)) / n
    pen = sum(s.sample(x, temperature=1.0, repetition_penalty=2.0, past_tokens={0: 1}) == 0 for _ in range(n)) / n
    more = sum(s.sample(x, temperature=1.0, repetition_penalty=2.0, past_tokens={0: 8}) == 0 for _ in range(n)) / n
    assert abs(base - 0.5) < 0.05 and pen < base - 0.1 and more < pen            # p^(1 + log2(count)) grows with count
    assert s.sample(x, temperature=0.0, repetition_penalty=2.0, past_tokens={0: 1}) == 1


def test_sampler_takes_the_reference_form_raw_fp16_bytes_and_a_vocabulary_size():
    row = np.full(12, -4.0, dtype=np.float16)
    row[5] = 3.0
    row[10] = 9.0                                             # padding beyond the vocabulary of 8: must not count
    data = row.tobytes()
    s = Sampler(seed=0)
    assert s.greedy(data, 8) == 5 and s.greedy(logits_bytes=data, vocab_size=8) == 5 and Sampler.greedy(data) == 10
    assert s.sample(data, vocab_size=8, temperature=0.0) == 5
    assert s.sample(logits_bytes=data, vocab_size=8, temperature=0.0) == 5
    assert s.sample(torch.from_numpy(row.astype(np.float32)), temperature=0.0, vocab_size=8) == 5
    with pytest.raises(ValueError, match="Expected 32 bytes"):
        s.greedy(data, 16)
    # past tokens as a plain set (the reference allows it): every member counts once
    x = torch.tensor([2.0, 2.0])
    n = 1500
    frac = sum(s.sample(x, temperature=1.0, repetition_penalty=2.0, past_tokens={0}) == 0 for _ in range(n)) / n
    assert frac < 0.4
