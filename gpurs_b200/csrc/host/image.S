/* Embeds the sm_100a kernel image (a fatbin produced by nvcc from csrc/kernels) into the library. */
    .section .rodata
    .balign 64
    .global gpurs_embedded_image
gpurs_embedded_image:
    .incbin GPURS_IMAGE_PATH
gpurs_embedded_image_end:
    .balign 8
    .global gpurs_embedded_image_size
gpurs_embedded_image_size:
    .quad gpurs_embedded_image_end - gpurs_embedded_image
    .section .note.GNU-stack,"",@progbits
