"""When the bucketed, overlapped gradient exchange is chosen over one exchange after backward."""
from chaoscontrol_b200.parallel import grad_overlap as G


def test_rule_follows_the_estimated_exposed_exchange(monkeypatch):
    monkeypatch.delenv("CCB_GRAD_OVERLAP", raising=False)
    small = 10_751_232 * 2                      # the 10.8 M-parameter model's bf16 payload
    assert not G.overlap_wanted(small, 2) and not G.overlap_wanted(small, 8)        # 0.03 ms / 0.2 ms of peer reads
    big = 57_690_624 * 2                        # the 57.7 M-parameter model
    assert not G.overlap_wanted(big, 2) and G.overlap_wanted(big, 4) and G.overlap_wanted(big, 8)
    assert not G.overlap_wanted(big, 1)
    # the threshold itself: payload * (ws - 1) / bandwidth against the minimum exposed time
    edge = int(G.OVERLAP_MIN_EXPOSED_S * G.PEER_BYTES_PER_S)
    assert not G.overlap_wanted(edge, 2) and G.overlap_wanted(edge + 1024, 2)


def test_environment_forces_either_way(monkeypatch):
    monkeypatch.setenv("CCB_GRAD_OVERLAP", "1")
    assert G.overlap_wanted(1024, 2)
    monkeypatch.setenv("CCB_GRAD_OVERLAP", "0")
    assert not G.overlap_wanted(1 << 40, 8)
