from kohakuwullm_b200.bench.abtest import admissible, loss_gap, noise_floor, windowed_gaps  # noqa: F401
from kohakuwullm_b200.bench.timing import (  # noqa: F401
    bench_ms, bench_peak_memory, bench_samples, cpu_enqueue_ms, device_op_counts, flush_l2, gpu_is_busy, graph_ms,
    measured_peaks, module_metrics, rel_error, stream_bandwidths, timing_profile, ulp_error,
)
from kohakuwullm_b200.data.synthetic import make_pack, make_packs  # noqa: F401
