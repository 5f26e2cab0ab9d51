"""Model zoo: the reference's transformer LM in RTP / TP / plain form, plus GPT-, Llama- and MoE-shaped LMs."""
