from .modeling_tusipel import NeuronTusipelForCausalLM, NeuronTusipelModel, TusipelInferenceConfig  # noqa: F401
