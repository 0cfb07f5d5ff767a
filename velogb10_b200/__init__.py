"""velogb10_b200: a Blackwell-datacenter (sm_100a) inference engine for hybrid GatedDeltaNet +
gated-GQA language models (dense and MoE) with NVFP4/FP8 weights, continuous batching, prefix
caching, lossless MTP speculation and tensor/expert parallelism over NVLink peer memory."""
__version__ = "0.1.0"
