"""Command-line tools: `estimate` (analytic model / memory / time + auto-parallel search), `tokenize`
(byte-BPE to NXTK shards); the process launcher `nexus-run` is a native executable built into ``bin/``."""
