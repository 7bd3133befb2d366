# Convenience targets (the reference drives its campaigns from scripts/Makefile; same names here).
PY ?= python
GPUS ?= 8
CLUSTER_NAME ?= local
PLATFORM ?= B200
export CLUSTER_NAME PLATFORM

.PHONY: bench_masks build test test-gpu bench cluster_profile bsa_train dense_train bsa_infer report plan fusion_table full_plans predict \
        figure6 figure7 figure8 figure9 figure10 figure11
DB ?= database/$(CLUSTER_NAME)/$(PLATFORM)
CONFIG ?= configs/stride.yaml

build:            ## compile the sm_100a kernel library in-tree (nvcc; works without a GPU)
	$(PY) -c "import __graft_entry__ as g; g.build()"

test:             ## CPU tests (planner, gloo executors, host logic of the fused path, model parity)
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu:         ## kernel and multi-GPU tests (multi-GPU ones skip on a single GPU)
	$(PY) -m pytest tests -q -m gpu

bench:            ## headline benchmark on $(GPUS) GPUs
	$(PY) -m ultraattn_b200.drivers.launch --gpus $(GPUS) -- bench.py --gpus $(GPUS)

cluster_profile:  ## kernel grid + link curves -> logs/m_configs (inputs of the cost model)
	$(PY) -m ultraattn_b200.drivers.cluster_profile --kernels --out logs/m_configs
	$(PY) -m ultraattn_b200.drivers.launch --gpus 2 -- -m ultraattn_b200.drivers.cluster_profile --comm --out logs/m_configs

bsa_train dense_train bsa_infer:   ## planning + profiling campaign of one experiment class
	$(PY) -m ultraattn_b200.drivers.launch --gpus $(GPUS) -- search_algo/task1_bsa.py --exp-class $@
	$(PY) -m ultraattn_b200.drivers.launch --gpus $(GPUS) -- search_algo/task2_bsa.py --exp-class $@

report:           ## figure tables from the profile database
	$(PY) -m ultraattn_b200.drivers.report --db $(DB)

# The reference's scripts/Makefile names its campaigns after the figures they feed; same names here.
figure7: bsa_train      ## block-sparse training patterns: campaign, then speed-ups over the baselines
	$(PY) -m ultraattn_b200.drivers.report --db $(DB)
figure8: dense_train    ## dense (full, causal) training
	$(PY) -m ultraattn_b200.drivers.report --db $(DB)
figure9: bsa_infer      ## star / streaming prefill
	$(PY) -m ultraattn_b200.drivers.report --db $(DB)
figure6:                ## end-to-end step times: 32 layers x (fwd + bwd) + a constant, from the database
	$(PY) -m ultraattn_b200.drivers.report --db $(DB) --e2e-layers 32 --e2e-const $(or $(E2E_CONST),0)
figure10:               ## strong and weak scalability across the rank counts in the database
	$(PY) -m ultraattn_b200.drivers.report --db $(DB) --scalability strong
	$(PY) -m ultraattn_b200.drivers.report --db $(DB) --scalability weak
figure11:               ## predicted against measured times (outlier share, R^2)
	$(PY) -m ultraattn_b200.drivers.report --db $(DB) --level intra --sim-accuracy
	$(PY) -m ultraattn_b200.drivers.report --db $(DB) --level inter --sim-accuracy

bench_masks:      ## token-level masks (causal, sliding window, prefix-LM, documents) on the kernels: error and time
	$(PY) -m ultraattn_b200.drivers.bench_masks

plan:             ## one configuration from a YAML file: plan, predicted time (add a launcher to run it)
	$(PY) -m ultraattn_b200.drivers.main --config $(CONFIG) --plan-only

fusion_table:     ## speed-up of fused x-by-y tiles over single tiles, from the machine profile
	$(PY) -m ultraattn_b200.drivers.fusion_evaluate --m-config ultraattn_b200/data/m_configs/$(PLATFORM)

full_plans:       ## all Y x X plans of full attention for $(GPUS) ranks into the plan database
	$(PY) -m ultraattn_b200.drivers.intra_attn_gen --cp $(GPUS)

predict:          ## cost-model predictions: fused runtime against the ring baselines for the named configs
	$(PY) -m ultraattn_b200.drivers.predict
