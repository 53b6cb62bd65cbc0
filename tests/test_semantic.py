"""Semantic layer: vocabulary encoding, text matching, targets, LSH retrieval."""
import json

import numpy as np
import pytest

from neuralfn_b200 import semantic as S


def test_encode_decode_and_matching():
    v = S.ConversationalVocabulary()
    assert v.vector_dim == v.num_vocab_dims + 1 and v.semantic_dim_names[-1] == S.TAXONOMY_HASH_NAME
    row = {"entity_type": "Software", "action": "repair", "domain": "technology", "semantic_signature": "sof_rep_tec"}
    vec = v.encode_row(row)
    back = v.decode_vector(vec)
    assert back["entity_type"] == "software" and back["action"] == "repair" and back["domain"] == "technology"
    assert 0.0 <= back[S.TAXONOMY_HASH_NAME] < 1.0
    topics = v.match_topics_in_text("Please repair the software before the deadline; daily life is complex.")
    assert topics["action"] == "repair" and topics["entity_type"] == "software" and topics["domain"] == "daily_life"
    assert topics["temporal"] == "deadline" and topics["property"] == "complex"


def test_targets_vectors_and_signature_are_deterministic():
    v = S.ConversationalVocabulary()
    t = S.build_semantic_targets_from_topics({"entity_type": "person", "action": "learn"}, vocab=v)
    assert t[v.dimension_to_expert["entity_type"]] == 0 and t[v.dimension_to_expert["domain"]] == S.SEMANTIC_IGNORE_INDEX
    assert S.build_semantic_signature(t, vocab=v) == "per_lea_non"
    assert t[-1] == S.signature_to_bucket("per_lea_non") == int(__import__("hashlib").md5(b"per_lea_non").hexdigest()[:8], 16) % 4096
    vec = S.semantic_targets_to_vectors(t, vocab=v)[0]
    assert vec[v.dimension_to_expert["entity_type"]] == -1.0 and vec[v.dimension_to_expert["domain"]] == 0.0
    r = S.semantic_targets_to_router_vectors(t, vocab=v)[0]
    assert r.shape == (v.num_vocab_dims,) and 0 <= r.min() and r.max() <= 1
    ids, tg = S.load_training_targets(50, vocab=v, seed=3)
    ids2, tg2 = S.load_training_targets(50, vocab=v, seed=3)
    assert np.array_equal(tg, tg2) and ((tg[:, :-1] >= 0).sum(1) == 2).all()
    with pytest.raises(ValueError):
        S.resolve_semantic_topics({"action": "teleport"}, vocab=v)


def test_external_vocabulary_file_and_lsh(tmp_path, monkeypatch):
    (tmp_path / "vocab_x.json").write_text(json.dumps({"vocabulary": {"entity_type": ["a b", "c"], "action": ["run"], "domain": ["d"]}}))
    monkeypatch.setenv("NFN_SEMANTIC_VOCAB_DIR", str(tmp_path))
    v = S.ConversationalVocabulary("vocab_x")
    assert v.match_topics_in_text("we saw A  B today")["entity_type"] == "a b"
    p = S.generate_synthetic_semantic_data(400, seed=1, out_dir=tmp_path)
    m = S.SemanticMatrix(p)
    h = m.build_hasher(tables=8, planes=6)
    q = m.vectors[17]
    ids, scores = h.query(q, k=400)
    assert 17 in ids.tolist() and scores[0] >= scores[-1]  # an indexed vector always meets itself in every table
    bi, bs = m.neighbors(q, k=3)
    assert abs(bs[0] - 1.0) < 1e-5 and np.allclose(m.vectors[bi[0]], q)
    assert h.get_projection_planes().shape == (8, 6, m.vectors.shape[1])
