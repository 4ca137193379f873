"""Running a quantized model: the fused decoder, graphed decode, and (later) tensor parallel."""
