// src/ptensor/tensor.rs, Tensor::attention (107-139): what changes.
//
//  * kv_head_num: K arrives permuted [batch, kv_head, seq, head_dim], so the KV-head count is
//    shape[1]; the snapshot passes shape[2], which is the sequence dimension (tensor.rs:131).
//  * the device operator also needs the cache's capacity and the largest chunk it will be given;
//    both are shapes this function already has: max_seq = k_tensor.shape[2] (rows per (sequence,
//    KV head) of the permuted K tensor) and max_interval = self.shape[0] (Q is
//    [sequence_chunk_size, batch, heads, head_dim]; sequence_chunk_size comes from
//    src/bin/main.rs:12-15 through Model::new).

        let operator = Operator::Attention(
            Attention::new(
                self.data,
                k_tensor.data,
                v_tensor.data,
                output_tensor.data,
                self.shape[1],
                self.shape[2],
                k_tensor.shape[1],          // was k_tensor.shape[2]
                self.shape[3],
                k_tensor.strides.clone(),
                inverse_sqrt_head,
            )
            .with_geometry(k_tensor.shape[2], self.shape[0]),   // max_seq, max_interval
        );
