"""The byte layout of the reference's per-layer state bank (src/runtime/state_residency.c:
44-54, 346-395: components [values, positions, auxiliary] at 8-byte aligned offsets of a
running cursor), restated by yvex_b200_kv_bank_layout. Integer arithmetic: exact."""
import ctypes as C

from clori_b200 import abi


def layout(library, components):
    array = (abi.KvBankComponent * len(components))(*[abi.KvBankComponent(*c) for c in components])
    spans = (abi.KvBankSpan * len(components))()
    total = abi.u64()
    ok = library.yvex_b200_kv_bank_layout(array, len(components), spans, C.byref(total))
    return ok, [(list(s.offset), list(s.bytes)) for s in spans], total.value


def test_dense_layer_bank(library):
    # one history component: 1000 rows of width 2 * 8 * 128 (K heads | V heads)
    ok, spans, total = layout(library, [(1, 1000, 2048, 0, 0)])
    assert ok == 1
    assert spans[0] == ([0, 1000 * 2048 * 4, 1000 * 2048 * 4 + 8000], [1000 * 2048 * 4, 8000, 0])
    assert total == 1000 * 2048 * 4 + 8000


def test_latent_layer_bank_with_rolling_components_and_odd_sizes(library):
    # local window (127 x 513 floats: an odd byte count), compressed history, main rolling state (3 x 5 floats)
    components = [(1, 127, 513, 0, 0), (1, 10, 512, 0, 0), (0, 0, 0, 15, 15)]
    ok, spans, total = layout(library, components)
    assert ok == 1
    cursor, expect = 0, []
    for history, capacity, width, kv, score in components:
        sizes = [capacity * width * 4, capacity * 8, 0] if history else [kv * 4, 0, score * 4]
        offsets = []
        for size in sizes:
            cursor = (cursor + 7) & ~7
            offsets.append(cursor)
            cursor += size
        expect.append((offsets, sizes))
    assert spans == expect and total == cursor
    assert spans[0][0][1] % 8 == 0 and (127 * 513 * 4) % 8 == 4      # the padding case is exercised


def test_refusals(library):
    assert layout(library, [(1, 1 << 62, 1 << 10, 0, 0)])[0] == 0      # overflow
    assert library.yvex_b200_kv_bank_layout(None, 1, None, None) == 0
