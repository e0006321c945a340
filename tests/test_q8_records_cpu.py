"""The Q8 KV record is a byte permutation of GGUF Q8_0 rows: every byte of the
rows lands at exactly one record offset and nothing else is written."""
import numpy as np

from clori_b200 import q8_records


def test_offsets_are_a_bijection_onto_the_record():
    k_lane, v_lane, k_scale, v_scale = q8_records.record_offsets()
    used = np.concatenate([k_lane.ravel(), v_lane.ravel(), k_scale.ravel(), k_scale.ravel() + 1,
                           v_scale.ravel(), v_scale.ravel() + 1])
    assert used.size == q8_records.RECORD_BYTES
    assert np.array_equal(np.sort(used), np.arange(q8_records.RECORD_BYTES))
    assert k_lane.max() < q8_records.V_LANES <= v_lane.min() and v_lane.max() < q8_records.K_SCALES
    assert k_scale.max() + 1 < q8_records.V_SCALES <= v_scale.min()


def test_pack_round_trips_through_the_offsets(oracle):
    rng = np.random.default_rng(1)
    tokens, heads = 150, 2
    values = rng.standard_normal((tokens, heads * 128)).astype(np.float32)
    k_rows = oracle.q8_0_encode_rows(values)
    v_rows = oracle.q8_0_encode_rows(values[::-1].copy())
    table = np.array([2, 0, 3], np.int32)
    records = q8_records.pack_records(k_rows, v_rows, heads, table, 4)
    k_lane, v_lane, k_scale, v_scale = q8_records.record_offsets()
    kb = k_rows.reshape(tokens, heads, 4, 34)
    for token in (0, 63, 64, 149):
        rec = records[table[token // 64], 1]
        t = token % 64
        assert np.array_equal(rec[k_lane[t]], kb[token, 1, :, 2:].reshape(128) ^ q8_records.LANE_BIAS)  # int8 + 128
        assert np.array_equal(rec[k_scale[t]], kb[token, 1, :, 0])
    assert not records[1].any()                      # pool block 1 is not in the table
    assert not records[3, 0][k_lane[22:].ravel()].any()  # slots beyond token 149 stay zero
