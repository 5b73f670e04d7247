"""The IUnifiedMemoryBuffer<T> members of UnifiedBuffer over real device memory (the bookkeeping itself is checked on
the CPU in test_unified_buffer_cpu.py): host views, Map, buffer-to-buffer copy, and a query that reads a buffer whose
newest data is still on the host."""
import numpy as np
import pytest

from dotcompute_b200 import AsComputeQueryable, BufferState, MapMode

pytestmark = pytest.mark.gpu


def test_host_views_map_and_device_copy(acc):
    x = np.arange(1000, dtype=np.float32)
    buf = acc.Memory.AllocateAndCopyAsync(x)
    assert np.array_equal(buf.AsReadOnlySpan(), x)
    buf.AsSpan()[:10] = -1.0                                   # newest data on the host
    assert buf.State is BufferState.HostDirty
    # the query reads the device copy: the pending change must be uploaded first
    assert AsComputeQueryable(buf, acc).Count("v => v < 0f") == 10
    with buf.MapRange(10, 5, MapMode.ReadWrite) as m:
        assert m.Span.tolist() == [10.0, 11.0, 12.0, 13.0, 14.0]
        m.Span[:] = -2.0
    assert AsComputeQueryable(buf, acc).Count("v => v < 0f") == 15
    dst = acc.Memory.AllocateAsync(1000, np.float32)
    buf.CopyToAsync(dst)
    assert np.array_equal(dst.ToArray(), buf.ToArray()) and dst.ToArray()[12] == -2.0
    out = acc.Memory.AllocateAsync(1000, np.float32)
    out.FillAsync(0.0)
    buf.CopyToBufferAsync(out, sourceOffset=990, destinationOffset=0, count=10)
    assert out.ToArray()[:10].tolist() == x[990:].tolist() and out.ToArray()[10] == 0.0
