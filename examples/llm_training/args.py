"""Command-line flags of the LLM trainers (counterpart of the reference's examples/llm_training/args.py)."""
import argparse
import os


def get_args():
    p = argparse.ArgumentParser()
    p.add_argument("--dataset", default="synthetic", help="'synthetic' or a .pt file holding a list of 1-D token tensors")
    p.add_argument("--length-dist", default="lognormal", choices=["lognormal", "longtail", "uniform"])
    p.add_argument("--minibatch_size", type=int, default=8, help="sequences per rank per minibatch")
    p.add_argument("--micro_batch_size", type=int, default=1)
    p.add_argument("--max_token_len", type=int, default=65536)
    p.add_argument("--limit_dataset_token_len", type=int, default=None)
    p.add_argument("--model_name", default="qwen2.5-1.5b")
    p.add_argument("--hf-checkpoint", default=None,
                   help="folder of a Hugging Face Llama / Qwen2 checkpoint (config.json + safetensors): its "
                        "architecture and weights replace --model_name and the seeded initialisation")
    p.add_argument("--save-hf-checkpoint", default=None,
                   help="after the last step, write the model to this folder in the Hugging Face layout")
    p.add_argument("--checkpoint-dir", default=None,
                   help="train_fsdp2.py: resume from the newest checkpoint in this folder if there is one, and save there")
    p.add_argument("--checkpoint-every", type=int, default=0,
                   help="save model + optimizer every N minibatches (0: only after the last one)")
    p.add_argument("--packing_method", default="DynamicDiffMicro",
                   choices=["None", "DynamicSameMicro", "DynamicDiffMicro", "LocalSort", "DebugUneven"])
    p.add_argument("--cost_model", default="linear", choices=["linear", "fit", "flops"])
    p.add_argument("--run_name", default="run")
    p.add_argument("--project_name", default="odc_b200")
    p.add_argument("--forward_only", action="store_true", default=os.environ.get("FORWARD_ONLY", "0") == "1")
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--lr", type=float, default=5e-4)
    p.add_argument("--activation-checkpointing", action="store_true")
    p.add_argument("--num-sequences", type=int, default=4096)
    p.add_argument("--loss-head", default="ce", choices=["ce", "logprobs"],
                   help="ce: fused linear + cross-entropy (one pass); logprobs: per-token log-probabilities, "
                        "loss = -(logp * loss_scale).sum() as the reference's trainers form it")
    p.add_argument("--cpu", action="store_true", help="CPU ranks over gloo and the host-shm heap (functional runs)")
    return p.parse_args()
