"""MLPerf-inference style offline harness (src/maxtext/inference/mlperf/)."""
